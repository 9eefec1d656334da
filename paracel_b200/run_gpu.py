"""GPU versions of the worker drivers: same executables, same JSON keys and the same output
files as ``run.py``, with the parameter-server shards in HBM and the device kernels doing the
work.  ``python -m paracel_b200.run <algorithm> ...`` dispatches here when the launcher was
started with ``--gpu`` (environment ``PCL_USE_GPU=1``) and the algorithm has a device path:
``mf``, ``pagerank``, ``kmeans``, ``lr`` (dgd), ``gLDA`` / ``lda``.

Inputs are the reference's text formats (matrix_factorization/mf.hpp:39-43,
pagerank/pr.hpp:55-57, kmeans/kmeans.hpp:68-74, lr.cpp:75-93, gLDA.hpp:190-203).  Every rank
reads the whole input (``paracel_loadall``), renumbers the ids densely and keeps the part that the
rank grid assigns to it; the dumps carry the original ids.
"""
from __future__ import annotations

import os
from typing import Dict, List

import numpy as np
import torch
import torch.distributed as dist

from .utils.ext import expand, str_split
from .utils.types import SENTINEL


def _all_lines(pattern) -> List[str]:
    out: List[str] = []
    for fn in expand(pattern):
        with open(fn) as f:
            out.extend(l.rstrip("\n").rstrip("\r") for l in f)
    return [l for l in out if l]


def _device(comm) -> torch.device:
    lr = int(os.environ.get("LOCAL_RANK", str(comm.get_rank())))
    torch.cuda.set_device(lr % max(torch.cuda.device_count(), 1))
    return torch.device("cuda", torch.cuda.current_device())


def mf_gpu(comm, info, pt):
    from .models.mf_gpu import MfSgdGpu, balanced_groups, grid_rank
    dev = _device(comm)
    rows = [str_split(l, " \t") for l in _all_lines(pt.check_parse("input", str))]
    uid = np.asarray([int(r[0]) for r in rows], dtype=np.int64)
    iid = np.asarray([int(r[1]) for r in rows], dtype=np.int64)
    val = np.asarray([float(r[-1]) for r in rows], dtype=np.float32)     # user item [date] rating
    unames, u = np.unique(uid, return_inverse=True)
    inames, i = np.unique(iid, return_inverse=True)
    u, i = torch.as_tensor(u, device=dev), torch.as_tensor(i, device=dev)
    r = torch.as_tensor(val, device=dev)
    ssp = bool(pt.get("ssp_switch", True))
    m = MfSgdGpu(len(unames), len(inames), k=int(pt.get("k", 80)), alpha=float(pt.get("alpha", 0.005)),
                 beta=float(pt.get("beta", 0.01)), rounds=int(pt.get("rounds", 1)),
                 staleness=int(pt.get("limit_s", 3)) if ssp else 0, ssp=ssp, device=dev)
    ug = balanced_groups(torch.bincount(u, minlength=len(unames)), m.npx, spread_above=0.25)
    ig = balanced_groups(torch.bincount(i, minlength=len(inames)), m.npy, spread_above=0.25)
    keep = grid_rank(u, i, ug, ig, m.npx, m.npy) == comm.get_rank()
    m.load_ratings(u[keep], i[keep], r[keep])
    m.init_parameters()
    m.fit()
    print("rmse:", m.rmse())
    m.dump_result(pt.parse("output", str), user_names=unames, item_names=inames)
    return m


def pagerank_gpu(comm, info, pt):
    from .models.pagerank_gpu import PageRankGpu
    dev = _device(comm)
    pairs = [str_split(l, ",") for l in _all_lines(pt.check_parse("input", str))]
    src = np.asarray([int(p[0]) for p in pairs], dtype=np.int64)
    dst = np.asarray([int(p[1]) for p in pairs], dtype=np.int64)
    names = np.unique(np.concatenate([src, dst[dst != SENTINEL]]))
    s = torch.as_tensor(np.searchsorted(names, src), device=dev)
    real = dst != SENTINEL
    d_idx = np.where(real, np.searchsorted(names, np.where(real, dst, names[0])), SENTINEL)
    d = torch.as_tensor(d_idx, device=dev)
    pr = PageRankGpu(len(names), float(pt.get("damping_factor", 0.85)), device=dev)
    # an edge lives on the owner of its target; "no out-link" markers on the owner of their source
    owner = torch.where(d == SENTINEL, pr.owner_of(s), pr.owner_of(torch.clamp(d, max=len(names) - 1)))
    mine = owner == comm.get_rank()
    pr.load_edges(s[mine], d[mine])
    pr.run(int(pt.get("rounds", 1)))
    pr.dump_result(pt.parse("output", str), names=names)
    return pr


def kmeans_gpu(comm, info, pt):
    from .models.kmeans_gpu import KMeansGpu
    from .ops.gemm import argmin_nt
    from .utils.dump import dump_dict_vector
    dev = _device(comm)
    ids, feats = [], []
    for l in _all_lines(pt.check_parse("input", str)):
        a, b = l.split("\t", 1)
        ids.append(a)
        feats.append([float(x) for x in b.split(",")])
    X = torch.as_tensor(np.asarray(feats, dtype=np.float32), device=dev)
    n, world, rank = X.shape[0], comm.get_size(), comm.get_rank()
    lo, hi = rank * n // world, (rank + 1) * n // world
    k = int(pt.get("kclusters", 2))
    km = KMeansGpu(k, X.shape[1], device=dev)
    km.load(X[lo:hi], init_centres=X[:k].clone())     # the first k rows seed the centres
    km.fit(int(pt.get("rounds", 1)))
    C = km.cluster_centres()
    _, arg = argmin_nt(X[lo:hi].contiguous(), C.contiguous(), precise=True)
    groups: Dict[int, List[str]] = {}
    for j, c in enumerate(arg.cpu().tolist()):
        groups.setdefault(int(c), []).append(ids[lo + j])
    parts = [groups]
    if world > 1:
        parts = [None] * world
        dist.all_gather_object(parts, groups)
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
    return km


def lr_gpu(comm, info, pt):
    """The ``dgd`` method (full-pass gradient with theta frozen, one bupdate per round) on the GPU."""
    from .models.linear_gpu import DenseLinearGpu
    from .utils.dump import dump_vector
    dev = _device(comm)
    rows = np.asarray([[float(x) for x in l.split(",")] for l in _all_lines(pt.check_parse("training_input", str))],
                      dtype=np.float32)
    n, world, rank = rows.shape[0], comm.get_size(), comm.get_rank()
    lo, hi = rank * n // world, (rank + 1) * n // world
    X = np.concatenate([np.ones((hi - lo, 1), dtype=np.float32), rows[lo:hi, :-1]], axis=1)   # bias column first
    y = rows[lo:hi, -1]
    m = DenseLinearGpu(X.shape[1], eta=float(pt.get("alpha", 0.002)) * n, beta=float(pt.get("beta", 0.1)),
                       device=dev)
    g = torch.Generator().manual_seed(0)
    m.load(torch.as_tensor(X), torch.as_tensor(y), theta0=torch.rand(X.shape[1], generator=g).to(dev))
    for _ in range(int(pt.get("rounds", 1))):
        m.step()
    m.step()                       # one more gradient evaluation gives the loss at the final theta
    print("final loss:", m.mean_loss())
    theta = m.weights().cpu().tolist()
    out = pt.parse("output", str)
    if rank == 0:
        os.makedirs(out, exist_ok=True)
        dump_vector(theta, os.path.join(out, "lr_theta_0"), sep="|")
    return m


def lda_gpu(comm, info, pt):
    from .models.lda_gpu import LdaGibbsGpu
    dev = _device(comm)
    docs = [str_split(l, " \t") for l in _all_lines(pt.check_parse("input", str))]
    vocab = sorted({w for d in docs for w in d})
    wid = {w: j for j, w in enumerate(vocab)}
    world, rank = comm.get_size(), comm.get_rank()
    lo, hi = rank * len(docs) // world, (rank + 1) * len(docs) // world
    mine = docs[lo:hi]
    ptr = np.zeros(len(mine) + 1, dtype=np.int64)
    np.cumsum([len(d) for d in mine], out=ptr[1:])
    words = np.asarray([wid[w] for d in mine for w in d], dtype=np.int32)
    K = int(pt.get("k_topics", 128))
    m = LdaGibbsGpu(len(vocab), K, pt.get("alpha", None), float(pt.get("beta", 0.01)),
                    iters=int(pt.get("iters", 10)), nbatch=1, staleness=0, device=dev)
    m.load_docs(torch.as_tensor(ptr, device=dev), torch.as_tensor(words, device=dev))
    ll = m.fit(with_loglik=bool(pt.get("debug", False)))
    if ll:
        print("log-likelihood:", ll[-1], "perplexity:", m.perplexity(ll[-1]))
    # top words of every topic, `<k>topic\t<word>:%f|...|` (gLDA.hpp:148, 174-180)
    ids = m.wt.owned_ids().cpu().numpy()
    counts = m.wt.shard[: len(ids)].cpu().numpy()
    parts = [(ids, counts)]
    if world > 1:
        parts = [None] * world
        dist.all_gather_object(parts, (ids, counts))
    if rank == 0:
        full = np.zeros((len(vocab), K), dtype=np.int64)
        for pi, pc in parts:
            full[pi] = pc
        beta, topk = float(pt.get("beta", 0.01)), int(pt.get("top_words", 10))
        tot = full.sum(0) + len(vocab) * beta
        outp = pt.parse("output", str)
        os.makedirs(os.path.dirname(outp) or ".", exist_ok=True)
        with open(outp + "0", "w") as f:
            for k in range(K):
                best = np.argsort(-full[:, k], kind="stable")[:topk]
                f.write(f"{k}topic\t" + "".join("%s:%f|" % (vocab[w], (full[w, k] + beta) / tot[k]) for w in best) + "\n")
    m._barrier()
    return m


GPU_ALGORITHMS = {"mf": mf_gpu, "pagerank": pagerank_gpu, "kmeans": kmeans_gpu, "lr": lr_gpu,
                  "gLDA": lda_gpu, "lda": lda_gpu}
