"""Worker bodies of the multi-GPU tests (run as child processes, one per GPU,
by ``paracel_b200.launch.local.LocalJob``)."""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


def symm_and_rows(comm, server_info):
    from paracel_b200.parallel.symm import SymmBuffer
    from paracel_b200.ps.tables import RowTable
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    # --- peer-visible buffer: everybody writes its rank into its own buffer, reads the peers'
    b = SymmBuffer(1024, torch.float32)
    b.local.fill_(float(rank + 1))
    torch.cuda.synchronize()
    comm.synchronize()
    out["peer_vals"] = [float(b.peer_view(r)[5].item()) for r in range(world)]
    comm.synchronize()
    b.free()
    # --- row table: pull rows owned by every rank, push weighted deltas, check owners
    rows, width = 1000, 128
    t = RowTable(rows, width, torch.float32)
    own = t.owned_ids()
    t.shard[: own.numel()] = own.to(torch.float32)[:, None] * 0.001 + torch.arange(width, device=dev)[None, :]
    torch.cuda.synchronize()
    comm.synchronize()
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    ids = torch.unique(torch.randint(0, rows, (400,), device=dev, generator=g))
    cur = torch.empty(ids.numel(), width, device=dev)
    old = torch.empty_like(cur)
    t.pull(ids, cur, old)
    torch.cuda.synchronize()
    exp = ids.to(torch.float32)[:, None] * 0.001 + torch.arange(width, device=dev)[None, :]
    out["pull_ok"] = bool(torch.allclose(cur, exp))
    comm.synchronize()
    cur += 1.0  # every holder adds one
    wgt = torch.full((ids.numel(),), 0.5, device=dev)
    t.push(ids, cur, old, wgt)
    torch.cuda.synchronize()
    comm.synchronize()
    # holders per row
    cnt = torch.zeros(rows, device=dev)
    cnt[ids] = 1.0
    dist.all_reduce(cnt)
    own_exp = own.to(torch.float32)[:, None] * 0.001 + torch.arange(width, device=dev)[None, :] \
        + 0.5 * cnt[own][:, None]
    out["push_ok"] = bool(torch.allclose(t.shard[: own.numel()], own_exp, atol=1e-5))
    comm.synchronize()
    t.free()
    # --- int rows + scalars
    ti = RowTable(64, 1024, torch.int32)
    idsi = torch.arange(0, 64, device=dev)
    one = torch.ones(64, 1024, dtype=torch.int32, device=dev)
    ti.push(idsi, one)
    torch.cuda.synchronize()
    comm.synchronize()
    got = torch.empty_like(one)
    ti.pull(idsi, got)
    torch.cuda.synchronize()
    out["int_ok"] = bool(torch.all(got == world))
    comm.synchronize()
    ti.free()
    return out


def ssp_clock(comm, server_info):
    """Rank 1 is slow; rank 0 may run at most `staleness` clocks ahead.  Then rank 1 stops
    committing (a flag that nothing sets) and rank 0's bounded wait reports a timeout."""
    from paracel_b200.parallel.ssp_device import DeviceSspClock, SspTimeout
    rank = comm.get_rank()
    c = DeviceSspClock(staleness=2, total_iters=100, timeout_s=0.5)
    comm.synchronize()
    ahead = []
    t0 = time.time()
    for it in range(6):
        c.wait()
        c.check()  # raises if the wait gave up
        torch.cuda.synchronize()
        mn = int(c.clocks[: c.world].min().item())
        ahead.append(c.clock - mn)
        if rank == 1:
            time.sleep(0.05)
        c.commit()
        torch.cuda.synchronize()
    comm.synchronize()
    res = {"max_ahead": max(ahead), "timeout": None}
    # withheld commit: rank 1 stays silent, rank 0 tries to go 3 more clocks
    if rank == 0:
        try:
            for it in range(4):
                c.wait()
                c.check()
                c.commit()
            res["timeout"] = "none"
        except SspTimeout as e:
            res["timeout"] = (e.expected, e.seen)
        # the context is still usable after the timed-out wait
        res["alive"] = float(torch.ones(4, device="cuda").sum().item())
    comm.synchronize()
    c.free()
    return res


def mf_train(comm, server_info, nu, ni, nnz, k, rounds, staleness):
    from paracel_b200.models.mf_gpu import MfSgdGpu, balanced_groups, grid_rank
    from paracel_b200.utils.synth import MfRatingStream
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = MfRatingStream(nu, ni, nnz, seed=5, device=dev)
    u, i, r = st.chunk_at(0)
    m = MfSgdGpu(nu, ni, k=k, alpha=0.005, beta=0.02, rounds=rounds, staleness=staleness,
                 ssp=staleness > 0, seed=3)
    cu = torch.bincount(u, minlength=nu)
    ci = torch.bincount(i, minlength=ni)
    ug, ig = balanced_groups(cu, m.npx, spread_above=0.25), balanced_groups(ci, m.npy, spread_above=0.25)
    keep = grid_rank(u, i, ug, ig, m.npx, m.npy) == rank
    m.load_ratings(u[keep], i[keep], r[keep])
    m.init_parameters()
    m.pull()
    r0 = m.rmse()
    m.fit()
    r1 = m.rmse()
    n_local = int(keep.sum().item())
    m.free()
    return {"rmse0": r0, "rmse1": r1, "nnz_local": n_local, "mu": m.mu}


def fused_gather_gemm(comm, server_info, N, K, M, kernel=None):
    """B is sharded by rows over the ranks; every rank multiplies its own A by the whole B."""
    from paracel_b200.ops.gemm import DenseReadGemm
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    Bfull = torch.randn(N, K, device=dev, generator=g)        # same on every rank
    g.manual_seed(1000 + rank)
    A = torch.randn(M, K, device=dev, generator=g)
    if kernel == "2sm-wide":        # 256 x 512 items of the pair kernel
        op = DenseReadGemm(N, K, kernel="2sm", wide=1)
    else:
        op = DenseReadGemm(N, K, kernel=kernel, wide=0)
    lo, hi = op.local_rows()
    op.shard[: hi - lo] = Bfull[lo:hi]
    torch.cuda.synchronize()
    comm.synchronize()
    out = {}
    for it in range(2):  # second call exercises the epoch logic
        C = op(A)
        torch.cuda.synchronize()
        op.check()
        ref = (A.double() @ Bfull.double().T).float()
        out[f"err{it}"] = float((C - ref).abs().max().item() / ref.abs().max().item())
        comm.synchronize()
    bn = (Bfull * Bfull).sum(1)
    mn, arg = op(A, argmin_bnorm=bn)
    torch.cuda.synchronize()
    op.check()
    d = bn[None, :].double() - 2 * (A.double() @ Bfull.double().T)
    chosen = d[torch.arange(M, device=dev), arg.long()]
    out["argmin_ok"] = bool(torch.all(chosen <= d.min(1).values + 0.05))
    comm.synchronize()
    op.free()
    return out


def dense_table_two_ranks(comm, server_info):
    """Reduce-scatter + handler across ranks without any host barrier between rounds."""
    from paracel_b200.ps.tables import DenseTable
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    L = 10007
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    theta0 = torch.randn(L, device=dev, generator=g)
    t = DenseTable(L, handler="prox_l1", lr=0.05, lam=0.3)
    t.write(theta0)
    torch.cuda.synchronize()
    comm.synchronize()
    exp = theta0.clone()
    ok = True
    for it in range(5):
        cur = t.read()
        ok = ok and bool(torch.allclose(cur, exp, atol=1e-5))
        ds = []
        for r in range(world):
            g.manual_seed(1000 * it + r)
            ds.append(torch.randn(L, device=dev, generator=g))
        t.delta().copy_(ds[rank])
        t.bupdate()
        w = exp - 0.05 * sum(ds)
        exp = torch.sign(w) * torch.clamp(w.abs() - 0.05 * 0.3, min=0)
    cur = t.read()
    torch.cuda.synchronize()
    t.check()
    ok = ok and bool(torch.allclose(cur, exp, atol=1e-5))
    comm.synchronize()
    t.free()
    return ok


def l1lr_and_pagerank_two_ranks(comm, server_info):
    """Sparse L1-LR and PageRank on 2 ranks give what 1 rank gives on the union of the data."""
    from paracel_b200.models.linear_gpu import SparseLinearGpu
    from paracel_b200.models.pagerank_gpu import PageRankGpu
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(21)
    n, F, k = 8000, 2048, 10
    cols = (torch.rand(n, k, device=dev, generator=g) ** 2 * F).long().clamp(max=F - 1)
    y = (torch.rand(n, device=dev, generator=g) < 0.5).float()
    lo, hi = rank * n // world, (rank + 1) * n // world
    m = SparseLinearGpu(F, eta=1.0, lam=1e-3, nbatch=1, hot_T=512)
    m.load(torch.arange(0, (hi - lo) * k + 1, k, device=dev, dtype=torch.int64),
           cols[lo:hi].reshape(-1).int().contiguous(), y[lo:hi])
    for _ in range(10):
        m.step()
    w = m.weights()
    torch.cuda.synchronize()
    m.table.check()
    th = torch.zeros(F, device=dev, dtype=torch.float64)
    for _ in range(10):
        r = y.double() - torch.sigmoid(th[cols].sum(1))
        gg = torch.zeros(F, device=dev, dtype=torch.float64)
        gg.index_add_(0, cols.reshape(-1), r[:, None].expand(-1, k).reshape(-1))
        wv = th + gg / n
        th = torch.sign(wv) * torch.clamp(wv.abs() - 1e-3 / n, min=0)
    ok_lr = bool(torch.allclose(w.double(), th, rtol=2e-3, atol=2e-4))
    comm.synchronize()
    m.free()
    # PageRank
    nv, ne = 4001, 50000
    g.manual_seed(22)
    src = torch.randint(0, nv, (ne,), device=dev, generator=g)
    dst = (torch.rand(ne, device=dev, generator=g) ** 2 * nv).long().clamp(max=nv - 1)
    pr = PageRankGpu(nv, 0.85)
    mine = pr.owner_of(dst) == rank
    pr.load_edges(src[mine], dst[mine])
    pr.run(12)
    outdeg = torch.bincount(src, minlength=nv).double()
    has = outdeg > 0
    ref = torch.where(has, torch.full((nv,), 1.0 / int(has.sum()), device=dev, dtype=torch.float64),
                      torch.zeros(nv, device=dev, dtype=torch.float64))
    for _ in range(12):
        c = torch.where(has, ref / outdeg.clamp(min=1), torch.zeros_like(ref))
        acc = torch.zeros(nv, device=dev, dtype=torch.float64)
        acc.index_add_(0, dst, c[src])
        ref = 0.15 + 0.85 * acc
    ok_pr = bool(torch.allclose(pr.ranks().double(), ref[pr.lo:pr.hi], rtol=1e-4, atol=1e-6))
    comm.synchronize()
    pr.free()
    return ok_lr, ok_pr


def kmeans_allreduce_lda_two_ranks(comm, server_info):
    """k-means (fused gather + arg-min GEMM, reduce-scatter of the sums), the one-launch
    all-reduce and the LDA sampler with sparse pulls / pushes on 2 ranks."""
    import numpy as np
    from paracel_b200.models.kmeans_gpu import KMeansGpu
    from paracel_b200.models.lda_gpu import LdaGibbsGpu
    from paracel_b200.ops.misc import DeviceAllReduce
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    ar = DeviceAllReduce()
    ok = True
    for it in range(4):
        x = torch.arange(6, dtype=torch.float64, device=dev) * (rank + 1) + it
        y = ar(x)
        torch.cuda.synchronize()
        exp = torch.arange(6, dtype=torch.float64, device=dev) * sum(r + 1 for r in range(world)) + it * world
        ok = ok and bool(torch.equal(y, exp))
    ar.check()
    out["allreduce"] = ok
    comm.synchronize()
    ar.free()
    # k-means: the same data split over the ranks must give the single-process Lloyd result
    g = torch.Generator(device=dev)
    g.manual_seed(31)
    k, d, n = 12, 6, 4000
    C0 = 5 * torch.randn(k, d, device=dev, generator=g)
    lab = torch.randint(0, k, (n,), device=dev, generator=g)
    X = C0[lab] + 0.4 * torch.randn(n, d, device=dev, generator=g)
    lo, hi = rank * n // world, (rank + 1) * n // world
    m = KMeansGpu(k, d)
    m.load(X[lo:hi], init_centres=X[:k].clone())
    m.fit(5)
    C = m.cluster_centres().double().cpu().numpy()
    Xn = X.double().cpu().numpy()
    Cr = Xn[:k].copy()
    for _ in range(5):
        a = ((Cr * Cr).sum(1)[None, :] - 2 * Xn @ Cr.T).argmin(1)
        for c in range(k):
            if (a == c).any():
                Cr[c] = Xn[a == c].mean(0)
    out["kmeans"] = bool(np.allclose(C, Cr, rtol=1e-3, atol=1e-3))
    comm.synchronize()
    m.free()
    # LDA: global bookkeeping stays exact with SSP staleness 2 and sparse pulls / pushes
    rng = np.random.default_rng(5)
    V, K, ndocs = 300, 128, 200
    ptr, words = [0], []
    for dd in range(ndocs):
        nn = int(rng.integers(20, 60))
        words.extend(rng.integers(0, V, nn).tolist())
        ptr.append(len(words))
    ptr, words = np.asarray(ptr), np.asarray(words)
    d0, d1 = rank * ndocs // world, (rank + 1) * ndocs // world
    lda = LdaGibbsGpu(V, K, iters=5, nbatch=3, staleness=2, seed=2)
    lda.load_docs(torch.tensor(ptr[d0:d1 + 1] - ptr[d0]), torch.tensor(words[ptr[d0]:ptr[d1]]))
    ll = lda.fit(with_loglik=True)
    tot = torch.tensor([int(lda.wt.shard.sum().item()), int(lda.ts.shard.sum().item())], device=dev)
    dist.all_reduce(tot)
    out["lda_counts"] = (int(tot[0]), int(tot[1]), len(words))
    out["lda_ll_up"] = ll[-1] > ll[0]
    colsum = lda.wt.shard.sum(0).clone()
    dist.all_reduce(colsum)
    nk = lda.ts.shard[0].clone() if rank == 0 else torch.zeros_like(lda.ts.shard[0])
    dist.all_reduce(nk)
    out["lda_consistent"] = bool(torch.equal(colsum.int(), nk.int()))
    comm.synchronize()
    lda.free()
    return out


def device_exchange_ranks(comm, server_info, pattern):
    """Every rank parses a different slice of one seeded triple list; after the device exchange
    each rank must hold exactly the triples that the placement function assigns to it, and the
    renumbering must agree with the union over its grid row / column."""
    from paracel_b200.load.device_exchange import DeviceExchange
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(123)
    n = 100_000
    A = torch.randint(0, 4000, (n,), device=dev, generator=g)
    B = torch.randint(0, 3000, (n,), device=dev, generator=g)
    W = torch.rand(n, device=dev, generator=g)
    lo, hi = rank * n // world, (rank + 1) * n // world
    ex = DeviceExchange(pattern)
    a2, b2, w2 = ex.exchange(A[lo:hi].contiguous(), B[lo:hi].contiguous(), W[lo:hi].contiguous())
    own = ex.owner(A, B) == rank
    key = lambda a, b, w: torch.sort(a.double() * 1e7 + b.double() * 1e3 + w.double()).values
    ok_triples = bool(torch.allclose(key(a2, b2, w2), key(A[own], B[own], W[own])))
    ri, ci, rm, cm = ex.index_mapping(a2, b2)
    rowc, colc = rank // ex.npy, rank % ex.npy
    all_owner = ex.owner(A, B)
    in_row = (all_owner // ex.npy) == rowc
    in_col = (all_owner % ex.npy) == colc
    ok_maps = bool(torch.equal(rm, torch.unique(A[in_row])) and torch.equal(cm, torch.unique(B[in_col])))
    ok_idx = bool(torch.equal(rm[ri], a2) and torch.equal(cm[ci], b2))
    return {"triples": ok_triples, "maps": ok_maps, "idx": ok_idx, "n": int(a2.numel())}


def paralg_device_backend_two_ranks(comm, server_info):
    """The public paralg calls on keys of device tables, from two ranks: a row written by one
    rank is read by the other out of the owner's HBM; updates of a dense key from both ranks give
    what the host parameter server gives for the same calls."""
    from paracel_b200.paralg import paralg
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    pt = paralg(server_info, comm, backend="gpu", device=dev)
    out = {}
    W = pt.paracel_row_table(1000, 8, prefix="W_", handler="mf_fac_updater")
    L = 10007
    pt.paracel_dense_table("theta", L, handler="lr_theta_update")
    row = [float(j) + 0.5 for j in range(8)]
    if rank == 0:
        pt.paracel_write("W_123", row)
    pt.paracel_sync()
    got = pt.paracel_read("W_123").tolist()
    out["row_read"] = got == row
    owner = 123 % world
    if rank == owner:
        out["row_in_owner_hbm"] = W.table.shard[123 // world].tolist() == row
    else:
        out["row_in_owner_hbm"] = float(W.table.shard[123 // world].abs().sum()) == 0.0
    # dense key: one-sided and collective updates from both ranks against the host server
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    theta0 = torch.randn(L, device=dev, generator=g)
    g.manual_seed(100 + rank)
    d1 = torch.randn(L, device=dev, generator=g)
    d2 = torch.randn(L, device=dev, generator=g)
    pt.paracel_write("theta", theta0)
    if rank == 0:
        pt.paracel_write("theta_host", theta0.double().cpu().tolist())
    pt.paracel_sync()
    pt.paracel_bupdate("theta", d1, "", "lr_theta_update")                    # one-sided, like the RPC
    pt.paracel_bupdate("theta_host", d1.double().cpu().tolist(), "", "lr_theta_update")
    pt.paracel_sync()
    pt.paracel_bupdate("theta", d2, "", "lr_theta_update", collective=True)   # fused reduce-scatter
    pt.paracel_bupdate("theta_host", d2.double().cpu().tolist(), "", "lr_theta_update")
    pt.paracel_sync()
    dev_val = pt.paracel_read("theta").double().cpu()
    host_val = torch.tensor(pt.paracel_read("theta_host"), dtype=torch.float64)
    out["dense_equals_host"] = bool(torch.allclose(dev_val, host_val, rtol=1e-5, atol=1e-5))
    # key batch from both ranks + filter view
    ids = torch.arange(rank, 1000, 7, device=dev)
    kb = pt.paracel_keys(W, ids)
    pt.paracel_bupdate_multi(kb, torch.ones(ids.numel(), 8, device=dev), "", "mf_fac_updater")
    pt.paracel_sync()
    allrows = pt.paracel_read_multi(pt.paracel_keys(W, torch.arange(1000, device=dev)))
    cnt = torch.zeros(1000, device=dev)
    for r in range(world):
        cnt[torch.arange(r, 1000, 7, device=dev)] += 1
    exp = cnt[:, None].expand(1000, 8).clone()
    exp[123] += torch.tensor(row, device=dev)
    out["batch_push"] = bool(torch.allclose(allrows, exp))
    d = pt.paracel_read_special("", "mf_W_filter")
    out["filter_view"] = len(d) == 1000 and d["W_123"] == exp[123].tolist()
    pt.paracel_check()
    pt.close()
    return out


def dense_linear_first_read_sees_theta0(comm, server_info):
    """A non-zero initial theta written collectively is what the first read returns on every
    rank, although one rank writes its slice a second later and nobody calls a barrier."""
    from paracel_b200.models.linear_gpu import DenseLinearGpu
    rank = comm.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    d = 4099
    g = torch.Generator().manual_seed(3)
    theta0 = torch.rand(d, generator=g).to(dev) + 1.0
    X = torch.randn(64, d, generator=g)
    y = (torch.rand(64, generator=g) < 0.5).float()
    m = DenseLinearGpu(d, eta=0.1)
    if rank == 1:
        time.sleep(1.0)
    m.load(X, y, theta0=theta0)
    first = m.paracel_read("theta").clone()
    ok = bool(torch.equal(first, theta0))
    m.step()
    m.paracel_sync()
    m.paracel_check()
    m.free()
    return ok


def suite_models_two_ranks(comm, server_info):
    """ALS, SVD, dense similarity and max-vertex-value on 2 ranks against fp64 NumPy oracles."""
    import numpy as np
    from paracel_b200.models.als_gpu import AlsGpu
    from paracel_b200.models.mvv_gpu import MvvGpu
    from paracel_b200.models.similarity_gpu import SimDenseGpu
    from paracel_b200.models.svd_gpu import SvdGpu
    rank, world = comm.get_rank(), comm.get_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    rng = np.random.default_rng(7)
    out = {}
    # ---- ALS: H rows live in the table, every rank solves the users u % world == rank
    nu, ni, k, lam = 300, 120, 24, 0.3
    H = rng.normal(size=(ni, k))
    uu = rng.integers(0, nu, 6000)
    ii = rng.integers(0, ni, 6000)
    _, first = np.unique(uu * ni + ii, return_index=True)
    uu, ii = uu[first], ii[first]
    rr = rng.uniform(1, 5, uu.size)
    als = AlsGpu(nu, ni, k, lam)
    mine = uu % world == rank
    flo, fhi = rank * ni // world, (rank + 1) * ni // world        # my slice of the factor file
    als.load(torch.tensor(uu[mine]), torch.tensor(ii[mine]), torch.tensor(rr[mine], dtype=torch.float32),
             torch.arange(flo, fhi), torch.tensor(H[flo:fhi], dtype=torch.float32))
    als.solve()
    Wd = als.paracel_read_multi(als.paracel_keys(als.W_tab, torch.arange(nu, device=dev)))[:, :k].double().cpu().numpy()
    ok = True
    for u in range(nu):
        sel = uu == u
        if not sel.any():
            continue
        Hs = H[ii[sel]]
        w = np.linalg.solve(Hs.T @ Hs + lam * np.eye(k), Hs.T @ rr[sel])
        ok = ok and np.allclose(Wd[u], w, rtol=2e-3, atol=2e-3)
    out["als"] = bool(ok)
    out["als_rmse"] = als.cal_rmse()
    als.free()
    # ---- SVD: low-rank + noise matrix, rows split over the ranks
    m, n, kk = 400, 90, 4
    A = (rng.normal(size=(m, kk)) * np.array([9.0, 6.0, 4.0, 2.5])) @ rng.normal(size=(kk, n)) + 0.01 * rng.normal(size=(m, n))
    A[rng.random((m, n)) < 0.3] = 0.0
    rows = np.arange(rank, m, world)
    sub = A[rows]
    nzr, nzc = np.nonzero(sub)
    ptr = np.zeros(rows.size + 1, dtype=np.int64)
    np.cumsum(np.bincount(nzr, minlength=rows.size), out=ptr[1:])
    svd = SvdGpu(n, kk, iters=25, oversample=8, seed=1)
    svd.load(torch.tensor(ptr), torch.tensor(nzc, dtype=torch.int32), torch.tensor(sub[nzr, nzc], dtype=torch.float32))
    svd.solve()
    S_ref = np.linalg.svd(A, compute_uv=False)[:kk]
    out["svd_sigma"] = bool(np.allclose(svd.sigma.numpy(), S_ref, rtol=2e-3))
    U = svd.U.double().cpu().numpy()
    V = svd.V.double().cpu().numpy()
    recon = (U * svd.sigma.numpy()[None, :]) @ V.T
    Ur, Sr, Vr = np.linalg.svd(A, full_matrices=False)
    best = (Ur[:, :kk] * Sr[:kk]) @ Vr[:kk]
    out["svd_recon"] = bool(np.abs(recon - best[rows]).max() < 2e-2 * np.abs(best).max())
    svd.free()
    # ---- dense similarity: every rank holds a block of the rows
    N, d, ktop = 500, 20, 5
    Xs = rng.normal(size=(N, d))
    ids = rng.permutation(10_000)[:N]
    lo, hi = rank * N // world, (rank + 1) * N // world
    sim = SimDenseGpu(d, ktop, simbar=-1.0)
    sim.load(torch.tensor(ids[lo:hi]), torch.tensor(Xs[lo:hi], dtype=torch.float32))
    sim.solve()
    Xn = Xs / np.linalg.norm(Xs, axis=1, keepdims=True)
    S = Xn @ Xn.T
    np.fill_diagonal(S, -np.inf)
    ok = True
    for a in range(lo, hi):
        want = np.argsort(-S[a])[:ktop]
        got = sim.result[int(ids[a])]
        ok = ok and [g_[0] for g_ in got] == [int(ids[j]) for j in want]
        ok = ok and np.allclose([g_[1] for g_ in got], S[a, want], atol=1e-4)
    out["sim_dense"] = bool(ok)
    sim.free()
    # ---- max vertex value: edges held by the owner of their source
    nv, ne = 400, 900
    es, ed = rng.integers(0, nv, ne), rng.integers(0, nv, ne)
    val = {int(v): float(v) for v in np.unique(es)}
    changed = True
    while changed:                                   # values flow along edges from source to target
        changed = False
        for a, b in zip(es.tolist(), ed.tolist()):
            if b in val and val[a] > val[b]:
                val[b] = val[a]
                changed = True
    mv = MvvGpu(nv)
    mine = es % world == rank
    mv.load_edges(torch.tensor(es[mine]), torch.tensor(ed[mine]))
    mv.solve()
    got = dict(zip(mv.lv.cpu().tolist(), mv.val.cpu().tolist()))
    out["mvv"] = all(got[v] == val[v] for v in got) and len(got) > 0
    mv.free()
    return out
