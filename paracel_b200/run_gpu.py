"""GPU versions of the worker drivers: same executables, same JSON keys and the same output
files as ``run.py``, with the parameter tables in HBM and the device kernels doing the work.
``python -m paracel_b200.run <algorithm> ...`` dispatches here when the launcher was started
with ``--gpu`` (environment ``PCL_USE_GPU=1``) and the algorithm has a device path: ``mf``,
``pagerank``, ``kmeans``, ``lr`` (dgd, ipm, downpour, agd), ``ridge``, ``lr_l1`` / ``lasso``,
``gLDA`` / ``lda``, ``als``, ``svd``, ``sim_dense``, ``sim_sparse``, ``mvv``.

Inputs are the reference's text formats (matrix_factorization/mf.hpp:39-43,
pagerank/pr.hpp:55-57, kmeans/kmeans.hpp:68-74, lr.cpp:75-93, gLDA.hpp:190-203,
als.hpp:103-131, sim_dense.hpp:84-101).  Loading follows the reference's loader
(include/ps.hpp:231-249, include/load/partition.hpp:57-86): every rank parses only its own
byte range of the input with the native parsers, the ranks agree on a dense numbering of the
ids they saw, and the parsed entries travel to the rank that owns them by one all-to-all on the
GPUs.  The dumps carry the original ids.
"""
from __future__ import annotations

import os
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ._core import core
from .utils.ext import expand, str_split
from .utils.types import SENTINEL


# ------------------------------------------------------------------ loading helpers
def _device(comm) -> torch.device:
    lr = int(os.environ.get("LOCAL_RANK", str(comm.get_rank())))
    torch.cuda.set_device(lr % max(torch.cuda.device_count(), 1))
    return torch.device("cuda", torch.cuda.current_device())


def _partition(comm, pattern):
    names = expand(pattern)
    if not names:
        raise FileNotFoundError(f"no input file matches {pattern!r}")
    return core().FilePartition(names, comm.get_size(), 1)


def _my_lines(comm, pattern) -> List[str]:
    """The lines of this rank's byte range of the input (line boundaries fixed up)."""
    r = comm.get_rank()
    return [l for l in _partition(comm, pattern).load_blocks(r, r + 1) if l]


def _my_triples(comm, pattern, seps: str, drop_fields: Sequence[int] = ()) -> Tuple[np.ndarray, ...]:
    """(a, b, w) arrays parsed natively from this rank's byte range: lines ``a<sep>b[<sep>w]``."""
    r = comm.get_rank()
    a, b, w, _ = _partition(comm, pattern).load_triples(r, r + 1, seps, False, 1, 1, list(drop_fields))
    return np.asarray(a, dtype=np.int64), np.asarray(b, dtype=np.int64), np.asarray(w, dtype=np.float32)


def _global_ids(comm, local: np.ndarray) -> np.ndarray:
    """Sorted union of the ids seen by all ranks (the dense numbering: id -> position)."""
    parts = comm.allgather(np.unique(local)) if comm.get_size() > 1 else [np.unique(local)]
    return np.unique(np.concatenate(parts)) if parts else np.zeros(0, dtype=np.int64)


def _exchange(comm, dev, dest: torch.Tensor, *cols: torch.Tensor) -> List[torch.Tensor]:
    """Send entry j of every column to rank ``dest[j]`` (one all-to-all per column on the GPUs);
    what arrives is ordered by source rank, then by the sender's order."""
    world = comm.get_size()
    if world == 1:
        return list(cols)
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    rc = torch.empty_like(counts)
    dist.all_to_all_single(rc, counts)
    sc, rcl = counts.tolist(), rc.tolist()
    out = []
    for c in cols:
        send = c[order].contiguous()
        recv = torch.empty(int(sum(rcl)), dtype=c.dtype, device=dev)
        dist.all_to_all_single(recv, send, rcl, sc)
        out.append(recv)
    return out


def _keep_last(key: torch.Tensor) -> torch.Tensor:
    """Indices of the last occurrence of every distinct key, in first-to-last order of position
    (a repeated input line overwrites the earlier one, as in the reference's graph containers,
    include/graph.hpp:226-232)."""
    n = key.numel()
    if n == 0:
        return torch.zeros(0, dtype=torch.int64, device=key.device)
    order = torch.argsort(key, stable=True)
    ks = key[order]
    last = torch.ones(n, dtype=torch.bool, device=key.device)
    last[:-1] = ks[1:] != ks[:-1]
    return torch.sort(order[last]).values


def _dense_rows(lines: List[str], seps: str = ",") -> np.ndarray:
    return np.asarray(core().parse_dense_rows(lines, seps), dtype=np.float32) if lines else np.zeros((0, 0), np.float32)


def _begin(m, pt=None):
    """Run options common to the device drivers: ``--metrics`` (or the config key ``metrics``)
    switches on metrics.jsonl and the phase trace, ``--resume DIR`` continues from a checkpoint
    that an earlier run of the same job wrote with ``--checkpoint DIR``."""
    if os.environ.get("PCL_METRICS", "0") == "1" or (pt is not None and pt.get("metrics", False)):
        m.paracel_enable_metrics()
    ck = os.environ.get("PCL_RESUME", "")
    if ck:
        from .utils import checkpoint as _ck
        if _ck.exists(ck):
            m.load_checkpoint(ck)
    return m


def _end(m):
    ck = os.environ.get("PCL_CHECKPOINT", "")
    if ck:
        m.save_checkpoint(ck)
    if m.timer is not None:
        m.dump_phase_trace()
    return m


# ------------------------------------------------------------------ drivers
def mf_gpu(comm, info, pt):
    from .models.mf_gpu import MfSgdGpu, balanced_groups, grid_rank
    dev = _device(comm)
    pattern = pt.check_parse("input", str)
    first = next(iter(_partition(comm, pattern).load_blocks(0, 1)), "")
    drop = [2] if len(str_split(first, " \t")) >= 4 else []          # user item [date] rating
    uid, iid, val = _my_triples(comm, pattern, " \t", drop)
    unames, inames = _global_ids(comm, uid), _global_ids(comm, iid)
    u = torch.as_tensor(np.searchsorted(unames, uid), device=dev)
    i = torch.as_tensor(np.searchsorted(inames, iid), device=dev)
    r = torch.as_tensor(val, device=dev)
    ssp = bool(pt.get("ssp_switch", True))
    m = MfSgdGpu(len(unames), len(inames), k=int(pt.get("k", 80)), alpha=float(pt.get("alpha", 0.005)),
                 beta=float(pt.get("beta", 0.01)), rounds=int(pt.get("rounds", 1)),
                 staleness=int(pt.get("limit_s", 3)) if ssp else 0, ssp=ssp, device=dev, comm=comm,
                 output=pt.parse("output", str), user_names=unames, item_names=inames,
                 update_funcs=pt.get("update_functions"))
    cu = torch.bincount(u, minlength=len(unames))
    ci = torch.bincount(i, minlength=len(inames))
    if comm.get_size() > 1:
        dist.all_reduce(cu)
        dist.all_reduce(ci)
    ug = balanced_groups(cu, m.npx, spread_above=0.25)
    ig = balanced_groups(ci, m.npy, spread_above=0.25)
    # spread rows are dealt by the other coordinate's id, so that a repeated (user, item) line
    # reaches the same rank as the line it overwrites
    dest = grid_rank(u, i, ug, ig, m.npx, m.npy, by_id=True)
    u, i, r = _exchange(comm, dev, dest, u, i, r)
    keep = _keep_last(u * len(inames) + i)
    m.load_ratings(u[keep], i[keep], r[keep])
    m.init_parameters()
    m.set_total_iters(m.rounds)
    _begin(m, pt)                  # a checkpoint replaces the fresh parameters and sets the clock
    m.paracel_sync()
    m.fit()
    print("rmse:", m.rmse())
    m.dump_result()
    return _end(m)


def pagerank_gpu(comm, info, pt):
    from .models.pagerank_gpu import PageRankGpu
    dev = _device(comm)
    src, dst, _ = _my_triples(comm, pt.check_parse("input", str), ",")
    names = _global_ids(comm, np.concatenate([src, dst[dst != SENTINEL]]))
    s = torch.as_tensor(np.searchsorted(names, src), device=dev)
    real = dst != SENTINEL
    d_idx = np.where(real, np.searchsorted(names, np.where(real, dst, names[0] if names.size else 0)), SENTINEL)
    d = torch.as_tensor(d_idx, device=dev)
    pr = PageRankGpu(len(names), float(pt.get("damping_factor", 0.85)), device=dev, comm=comm,
                     output=pt.parse("output", str))
    # an edge lives on the owner of its target; "no out-link" markers on the owner of their source
    owner = torch.where(d == SENTINEL, pr.owner_of(s), pr.owner_of(torch.clamp(d, max=max(len(names) - 1, 0))))
    s, d = _exchange(comm, dev, owner, s, d)
    # a repeated line is one edge: the reference keeps adj[v][w] (include/graph.hpp:226-232)
    keep = _keep_last(s * (SENTINEL + 1) + d)
    pr.load_edges(s[keep], d[keep])
    _begin(pr, pt)
    pr.run(max(0, int(pt.get("rounds", 1)) - pr.it))
    pr.dump_result(pt.parse("output", str), names=names)
    return _end(pr)


def kmeans_gpu(comm, info, pt):
    from .models.kmeans_gpu import KMeansGpu
    from .ops.gemm import argmin_nt
    from .utils.dump import dump_dict_vector
    dev = _device(comm)
    ids, feats = [], []
    for l in _my_lines(comm, pt.check_parse("input", str)):
        a, b = l.split("\t", 1)
        ids.append(a)
        feats.append(b)
    Xn = _dense_rows(feats)
    dim = torch.tensor([Xn.shape[1] if Xn.size else 0], device=dev)
    if comm.get_size() > 1:
        dist.all_reduce(dim, op=dist.ReduceOp.MAX)
    X = torch.as_tensor(Xn, device=dev).reshape(-1, int(dim.item()))
    world, rank = comm.get_size(), comm.get_rank()
    k = int(pt.get("kclusters", 2))
    km = KMeansGpu(k, X.shape[1], device=dev, comm=comm, output=pt.parse("output", str))
    km.load(X)                                   # the first k rows of worker 0 seed the centres
    _begin(km, pt)
    km.fit(int(pt.get("rounds", 1)))
    C = km.cluster_centres()
    groups: Dict[int, List[str]] = {}
    if X.shape[0]:
        _, arg = argmin_nt(X.contiguous(), C.contiguous(), precise=True)
        for j, c in enumerate(arg.cpu().tolist()):
            groups.setdefault(int(c), []).append(ids[j])
    parts = comm.allgather(groups) if world > 1 else [groups]
    out = pt.parse("output", str)
    if rank == 0:
        os.makedirs(out, exist_ok=True)
        merged: Dict[int, List[str]] = {}
        for p in parts:
            for c, v in p.items():
                merged.setdefault(c, []).extend(v)
        with open(os.path.join(out, "kmeans_0"), "w") as f:
            for c in sorted(merged):
                f.write(f"{c}\t{'|'.join(merged[c])}\n")
        dump_dict_vector({c: C[c].cpu().tolist() for c in range(k)}, os.path.join(out, "centers_0"))
    km._barrier()
    return _end(km)


def _linear_data(comm, pt, dev):
    rows = _dense_rows(_my_lines(comm, pt.check_parse("training_input", str)))
    n_local = rows.shape[0]
    d = torch.tensor([rows.shape[1] if rows.size else 0, n_local], device=dev)
    tot = d.clone()
    if comm.get_size() > 1:
        dmax = d.clone()
        dist.all_reduce(dmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot)
        d[0] = dmax[0]
    ncol = int(d[0].item())
    rows = rows.reshape(-1, ncol)
    X = np.concatenate([np.ones((n_local, 1), dtype=np.float32), rows[:, :-1]], axis=1)   # bias column first
    return torch.as_tensor(X), torch.as_tensor(rows[:, -1].copy()), int(tot[1].item())


def _linear_gpu(comm, info, pt, logistic: bool, dump_name: str):
    """``lr`` / ``ridge``: ``dgd`` is one full-pass gradient and one collective bupdate per round;
    ``ipm`` (default), ``downpour`` and ``agd`` are the reference's asynchronous methods with
    one-sided updates (lr.cpp:154-299)."""
    from .models.linear_gpu import DenseLinearGpu
    from .utils.dump import dump_vector
    dev = _device(comm)
    X, y, n = _linear_data(comm, pt, dev)
    alpha, beta = float(pt.get("alpha", 0.002)), float(pt.get("beta", 0.1))
    method = pt.get("method", "ipm")
    m = DenseLinearGpu(X.shape[1], eta=alpha * n, beta=beta, logistic=logistic, device=dev, comm=comm,
                       output=pt.parse("output", str))
    g = torch.Generator().manual_seed(0)
    m.load(X, y, theta0=torch.rand(X.shape[1], generator=g).to(dev))
    rounds = int(pt.get("rounds", 1))
    if method == "dgd":
        for _ in range(rounds):
            m.step()
    else:
        m.fit_async(method, rounds, alpha=alpha * float(pt.get("batch", 64)), batch=int(pt.get("batch", 64)))
    m.step()                       # one more gradient evaluation gives the loss at the final theta
    print("final loss:", m.mean_loss())
    theta = m.weights().cpu().tolist()
    out = pt.parse("output", str)
    if comm.get_rank() == 0:
        os.makedirs(out, exist_ok=True)
        dump_vector(theta, os.path.join(out, dump_name), sep="|")
    return m


def lr_gpu(comm, info, pt):
    return _linear_gpu(comm, info, pt, True, "lr_theta_0")


def ridge_gpu(comm, info, pt):
    return _linear_gpu(comm, info, pt, False, "ridge_theta_0")


def l1_gpu(comm, info, pt, logistic: bool = True):
    """Sparse L1-regularised logistic regression (``lr_l1``) / Lasso by proximal gradient with the
    prox-L1 handler applied at the owners of the weight shards.  Input: the dense CSV of the
    serial tools (``f1,...,fk,label``; tool/lr_l1_serial.cpp:100-120) or sparse lines
    ``label i:v i:v ...``.  The objective is ``sum_i loss_i + lambda * |w|_1`` (``lambda`` weighs
    the summed loss, as in the serial tools); ``eta`` is the step on the mean gradient.  Dumps
    ``lr_l1_weight_0`` / ``lasso_weight_0``."""
    from .models.linear_gpu import SparseLinearGpu
    from .utils.dump import dump_vector
    dev = _device(comm)
    lines = _my_lines(comm, pt.check_parse("input", str) if pt.get("input") else pt.check_parse("training_input", str))
    if lines and ":" in lines[0]:
        ptr, cols, vals, ys = [0], [], [], []
        for l in lines:
            f = str_split(l, " \t")
            ys.append(float(f[0]))
            for it in f[1:]:
                c, v = it.split(":")
                cols.append(int(c))
                vals.append(float(v))
            ptr.append(len(cols))
        F_local = (max(cols) + 1) if cols else 0
        row_ptr, cols_t = torch.tensor(ptr, dtype=torch.int64), torch.tensor(cols, dtype=torch.int32)
        vals_t, y = torch.tensor(vals, dtype=torch.float32), torch.tensor(ys, dtype=torch.float32)
    else:
        rows = torch.as_tensor(_dense_rows(lines))
        F_local = max(rows.shape[1] - 1, 0) if rows.numel() else 0
        Xd = rows[:, :-1] if rows.numel() else torch.zeros(0, 0)
        y = rows[:, -1].clone() if rows.numel() else torch.zeros(0)
        nzr, nzc = torch.nonzero(Xd, as_tuple=True)
        row_ptr = torch.zeros(Xd.shape[0] + 1, dtype=torch.int64)
        row_ptr[1:] = torch.cumsum(torch.bincount(nzr, minlength=Xd.shape[0]), 0)
        cols_t, vals_t = nzc.to(torch.int32), Xd[nzr, nzc]
    F = torch.tensor([F_local], device=dev)
    if comm.get_size() > 1:
        dist.all_reduce(F, op=dist.ReduceOp.MAX)
    F = int(F.item())
    if logistic:
        y = (y > 0).float()                          # labels {0,1} (or {-1,+1}) -> {0,1}
    m = SparseLinearGpu(F, eta=float(pt.get("eta", 0.5)), lam=float(pt.get("lambda", 1e-6)), logistic=logistic,
                        l1=True, device=dev, comm=comm, output=pt.parse("output", str),
                        nbatch=int(pt.get("nbatch", 1)))
    m.load(row_ptr, cols_t, y, vals_t)
    for _ in range(int(pt.get("rounds", 100))):
        m.epoch()
    print("loss:", m.mean_loss(), "nnz(w):", m.nnz_weights())
    w = m.weights().cpu().tolist()
    out = pt.parse("output", str)
    if comm.get_rank() == 0:
        os.makedirs(out, exist_ok=True)
        dump_vector(w, os.path.join(out, "lr_l1_weight_0" if logistic else "lasso_weight_0"), sep="|")
    m.paracel_sync()
    return m


def lasso_gpu(comm, info, pt):
    return l1_gpu(comm, info, pt, logistic=False)


def lda_gpu(comm, info, pt):
    from .models.lda_gpu import LdaGibbsGpu
    dev = _device(comm)
    docs = [str_split(l, " \t") for l in _my_lines(comm, pt.check_parse("input", str))]
    world, rank = comm.get_size(), comm.get_rank()
    local_vocab = sorted({w for d in docs for w in d})
    vocab = sorted(set().union(*comm.allgather(local_vocab))) if world > 1 else local_vocab
    wid = {w: j for j, w in enumerate(vocab)}
    ptr = np.zeros(len(docs) + 1, dtype=np.int64)
    np.cumsum([len(d) for d in docs], out=ptr[1:])
    words = np.asarray([wid[w] for d in docs for w in d], dtype=np.int64)
    K = int(pt.get("k_topics", 128))
    m = LdaGibbsGpu(len(vocab), K, pt.get("alpha", None), float(pt.get("beta", 0.01)),
                    iters=int(pt.get("iters", 10)), nbatch=1, staleness=0, device=dev, comm=comm)
    m.load_docs(torch.as_tensor(ptr, device=dev), torch.as_tensor(words, device=dev))
    _begin(m, pt)
    ll = m.fit(with_loglik=bool(pt.get("debug", False)))
    if ll:
        print("log-likelihood:", ll[-1], "perplexity:", m.perplexity(ll[-1]))
    # top words of every topic, `<k>topic\t<word>:%f|...|` (gLDA.hpp:148, 174-180): worker 0 reads
    # the whole word-topic table out of the owners' HBM
    if rank == 0:
        rows = torch.arange(len(vocab), dtype=torch.int64, device=dev)
        full = m.paracel_read_multi(m.paracel_keys(m.wt_tab, rows), use_cache=False, ssp_wait=False).cpu().numpy().astype(np.int64)
        beta, topk = float(pt.get("beta", 0.01)), int(pt.get("top_words", 10))
        tot = full.sum(0) + len(vocab) * beta
        outp = pt.parse("output", str)
        os.makedirs(os.path.dirname(outp) or ".", exist_ok=True)
        with open(outp + "0", "w") as f:
            for k in range(K):
                best = np.argsort(-full[:, k], kind="stable")[:topk]
                f.write(f"{k}topic\t" + "".join("%s:%f|" % (vocab[w], (full[w, k] + beta) / tot[k]) for w in best) + "\n")
    m._barrier()
    return _end(m)


def als_gpu(comm, info, pt):
    """Ratings ``u,i,r`` partitioned by user (``fmap``), item factors ``id\\tf1|f2|...`` read in
    byte ranges and written to the owners of their rows; dumps ``W_<rank>``."""
    from .models.als_gpu import AlsGpu
    dev = _device(comm)
    world = comm.get_size()
    uid, iid, val = _my_triples(comm, pt.check_parse("rating_input", str), ",")
    fid, frows = [], []
    for l in _my_lines(comm, pt.check_parse("factor_input", str)):
        a, b = l.split("\t", 1)
        fid.append(int(a))
        frows.append(b)
    fac = _dense_rows(frows, "|")
    kdim = torch.tensor([fac.shape[1] if fac.size else 0], device=dev)
    if world > 1:
        dist.all_reduce(kdim, op=dist.ReduceOp.MAX)
    k = int(kdim.item())
    unames = _global_ids(comm, uid)
    inames = _global_ids(comm, np.asarray(fid, dtype=np.int64))
    if iid.size and not np.all(np.isin(iid, inames)):
        raise RuntimeError("Data error: rating data and factor data is not consistent.")
    u = torch.as_tensor(np.searchsorted(unames, uid), device=dev)
    i = torch.as_tensor(np.searchsorted(inames, iid), device=dev)
    r = torch.as_tensor(val, device=dev)
    u, i, r = _exchange(comm, dev, u % world, u, i, r)
    keep = _keep_last(u * max(len(inames), 1) + i)
    m = AlsGpu(len(unames), len(inames), k, float(pt.get("lambda", 0.1)), device=dev, comm=comm,
               output=pt.parse("output", str), user_names=unames, item_names=inames)
    m.load(u[keep], i[keep], r[keep],
           torch.as_tensor(np.searchsorted(inames, np.asarray(fid, dtype=np.int64)), device=dev),
           torch.as_tensor(fac.reshape(-1, k), device=dev))
    if pt.get("validate_input"):
        # the validate driver (als_validate_driver.cpp:56-86): sweep the lambdas, report the train
        # and the validation RMSE over the pairs whose user and item are known
        vu, vi, vr = _my_triples(comm, pt.get("validate_input"), ",")
        known = np.isin(vu, unames) & np.isin(vi, inames)
        vu_t = torch.as_tensor(np.searchsorted(unames, vu[known]), device=dev)
        vi_t = torch.as_tensor(np.searchsorted(inames, vi[known]), device=dev)
        vr_t = torch.as_tensor(vr[known], device=dev)
        for lam in pt.get("lambdas", [m.lam]):
            m.solve(float(lam))
            train = m.cal_rmse()
            sse, cnt = m.validate_sse(vu_t, vi_t, vr_t)
            tot = torch.tensor([sse, cnt], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(tot)
            if comm.get_rank() == 0:
                print(f"lambda {lam}: train rmse {train} validate rmse {float((tot[0] / tot[1].clamp(min=1)).sqrt())}")
    else:
        m.solve()
        print("rmse:", m.cal_rmse())
    m.dump_result()
    return m


def svd_gpu(comm, info, pt):
    """Triples ``row,col,val`` partitioned by row; dumps SIGMA_0, V_0 and U_<rank>."""
    from .models.svd_gpu import SvdGpu
    dev = _device(comm)
    world = comm.get_size()
    a, b, w = _my_triples(comm, pt.check_parse("input", str), ",")
    rnames, cnames = _global_ids(comm, a), _global_ids(comm, b)
    ra = torch.as_tensor(np.searchsorted(rnames, a), device=dev)
    cb = torch.as_tensor(np.searchsorted(cnames, b), device=dev)
    wv = torch.as_tensor(w, device=dev)
    ra, cb, wv = _exchange(comm, dev, ra % world, ra, cb, wv)
    keep = _keep_last(ra * max(len(cnames), 1) + cb)
    ra, cb, wv = ra[keep], cb[keep], wv[keep]
    rows, rl = torch.unique(ra, return_inverse=True)
    order = torch.argsort(rl, stable=True)
    ptr = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=dev)
    ptr[1:] = torch.cumsum(torch.bincount(rl, minlength=rows.numel()), 0)
    m = SvdGpu(len(cnames), int(pt.parse("k")), iters=int(pt.get("iters", 20)), device=dev, comm=comm,
               output=pt.parse("output", str), update_function=pt.get("update_function", "svd_updater"))
    m.load(ptr, cb[order].to(torch.int32), wv[order])
    m.solve()
    m.dump_result(row_names=[int(rnames[j]) for j in rows.cpu().tolist()], col_names=cnames.tolist())
    return m


def sim_dense_gpu(comm, info, pt):
    from .models.similarity_gpu import SimDenseGpu
    dev = _device(comm)

    def load(pattern):
        ids, feats = [], []
        for l in _my_lines(comm, pattern):
            a, b = l.split(",", 1)
            ids.append(int(a))
            feats.append(b)
        return torch.tensor(ids, dtype=torch.int64), torch.as_tensor(_dense_rows(feats))
    a = pt.get("input") or pt.get("input_a")
    b = pt.get("input_b") or a
    ids_a, A = load(a)
    ids_b, B = (ids_a, A) if b == a else load(b)
    dim = torch.tensor([A.shape[1] if A.numel() else 0, B.shape[1] if B.numel() else 0], device=dev)
    if comm.get_size() > 1:
        dist.all_reduce(dim, op=dist.ReduceOp.MAX)
    d = int(dim.max().item())
    m = SimDenseGpu(d, int(pt.get("topk", 20)), float(pt.get("simbar", 0.0)), device=dev, comm=comm,
                    output=pt.parse("output", str))
    m.load(ids_a, A.reshape(-1, d), ids_b, B.reshape(-1, d))
    m.solve()
    m.dump_result()
    return m


def sim_sparse_gpu(comm, info, pt):
    from .models.similarity_gpu import SimSparseGpu
    dev = _device(comm)
    world = comm.get_size()
    a, b, w = _my_triples(comm, pt.check_parse("input", str), ",")
    if pt.get("format", "fsv") == "sfv":
        a, b = b, a
    rnames, cnames = _global_ids(comm, a), _global_ids(comm, b)
    ra = torch.as_tensor(np.searchsorted(rnames, a), device=dev)
    cb = torch.as_tensor(np.searchsorted(cnames, b), device=dev)
    wv = torch.as_tensor(w, device=dev)
    ra, cb, wv = _exchange(comm, dev, ra % world, ra, cb, wv)
    keep = _keep_last(ra * max(len(cnames), 1) + cb)
    ra, cb, wv = ra[keep], cb[keep], wv[keep]
    rows, rl = torch.unique(ra, return_inverse=True)
    m = SimSparseGpu(len(cnames), int(pt.get("topk", 20)), float(pt.get("sim_bar", 0.0)), device=dev,
                     comm=comm, output=pt.parse("output", str))
    m.load_triples(torch.as_tensor(rnames, device=dev)[rows], rl, cb, wv)
    m.solve()
    m.dump_result()
    return m


def mvv_gpu(comm, info, pt):
    from .models.mvv_gpu import MvvGpu
    dev = _device(comm)
    world = comm.get_size()
    src, dst, _ = _my_triples(comm, pt.check_parse("input", str), ",")
    names = _global_ids(comm, np.concatenate([src, dst]))
    s = torch.as_tensor(np.searchsorted(names, src), device=dev)
    d = torch.as_tensor(np.searchsorted(names, dst), device=dev)
    s, d = _exchange(comm, dev, s % world, s, d)
    keep = _keep_last(s * max(len(names), 1) + d)
    m = MvvGpu(len(names), device=dev, comm=comm, output=pt.parse("output", str), names=names.tolist(),
               update_func=pt.get("update_func", "max_updater"))
    m.load_edges(s[keep], d[keep])
    m.solve()
    m.dump_result()
    return m


GPU_ALGORITHMS = {"mf": mf_gpu, "pagerank": pagerank_gpu, "kmeans": kmeans_gpu, "lr": lr_gpu,
                  "ridge": ridge_gpu, "lr_l1": l1_gpu, "lasso": lasso_gpu, "gLDA": lda_gpu, "lda": lda_gpu,
                  "als": als_gpu, "als_validate": als_gpu, "svd": svd_gpu, "sim_dense": sim_dense_gpu, "ab_sim_dense": sim_dense_gpu,
                  "sim_sparse": sim_sparse_gpu, "mvv": mvv_gpu}
