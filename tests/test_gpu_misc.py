"""Batched ALS solve, k-means, top-k merge, Gram and the one-launch all-reduce on one GPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k", [8, 32, 50, 128])
def test_als_batched_solve_matches_numpy(k):
    from paracel_b200.ops.als import als_solve
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(k)
    ni, nu = 500, 300
    H = torch.randn(ni, k, device=dev, generator=g)
    cnt = torch.randint(1, 40, (nu,), device=dev, generator=g)
    cnt[0] = 0                      # a user without ratings keeps a zero factor
    cnt[5] = 9000                   # a heavy user is split over several CTAs
    ptr = torch.zeros(nu + 1, dtype=torch.int64, device=dev)
    ptr[1:] = torch.cumsum(cnt, 0)
    nnz = int(ptr[-1])
    idx = torch.randint(0, ni, (nnz,), device=dev, generator=g).int()
    r = torch.randn(nnz, device=dev, generator=g)
    lam = 0.5
    W = als_solve(ptr, idx, r, H, lam, seg_len=1024)
    torch.cuda.synchronize()
    Hn, pn, idn, rn = H.double().cpu().numpy(), ptr.cpu().numpy(), idx.cpu().numpy(), r.double().cpu().numpy()
    for u in (0, 1, 5, 77, 299):
        Hs = Hn[idn[pn[u]:pn[u + 1]]]
        if Hs.shape[0] == 0:
            assert float(W[u].abs().sum()) == 0.0
            continue
        ref = np.linalg.solve(Hs.T @ Hs + lam * np.eye(k), Hs.T @ rn[pn[u]:pn[u + 1]])
        assert np.allclose(W[u].cpu().numpy(), ref, rtol=2e-3, atol=2e-4), u


def test_kmeans_gpu_matches_numpy_lloyd():
    from paracel_b200.models.kmeans_gpu import KMeansGpu
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(7)
    k, d, n = 16, 10, 6000
    C0 = 6 * torch.randn(k, d, device=dev, generator=g)
    lab = torch.randint(0, k, (n,), device=dev, generator=g)
    X = C0[lab] + 0.5 * torch.randn(n, d, device=dev, generator=g)
    m = KMeansGpu(k, d, device=dev)
    m.load(X)
    m.fit(6)
    C = m.cluster_centres().double().cpu().numpy()
    Xn = X.double().cpu().numpy()
    Cr = Xn[:k].copy()
    for _ in range(6):
        a = ((Cr * Cr).sum(1)[None, :] - 2 * Xn @ Cr.T).argmin(1)
        for c in range(k):
            if (a == c).any():
                Cr[c] = Xn[a == c].mean(0)
    assert np.allclose(C, Cr, rtol=1e-3, atol=1e-3)
    m.free()


@pytest.mark.parametrize("n,d,k", [(5003, 128, 37), (4001, 64, 5), (3000, 256, 100), (2500, 512, 9),
                                   (3001, 10, 7), (2000, 516, 3), (3, 128, 2)])
def test_kmeans_accumulate_matches_index_add(n, d, k):
    """Per-cluster sums and counts (vector-reduction kernel for d % 4 == 0 and d <= 512, the scalar
    kernel otherwise) against a plain fp64 index_add."""
    from paracel_b200.ops.misc import kmeans_accumulate
    g = torch.Generator(device="cuda").manual_seed(n + d)
    X = torch.randn(n, d, device="cuda", generator=g)
    assign = torch.randint(0, k, (n,), device="cuda", generator=g, dtype=torch.int32)
    sums = torch.zeros(k, d, device="cuda")
    counts = torch.zeros(k, device="cuda")
    kmeans_accumulate(X, assign, sums, counts)
    ref = torch.zeros(k, d, device="cuda", dtype=torch.float64).index_add_(0, assign.long(), X.double())
    cnt = torch.bincount(assign.long(), minlength=k).double()
    assert torch.equal(counts.double(), cnt)
    assert (sums.double() - ref).abs().max().item() < 1e-3


@pytest.mark.parametrize("rows,width,n", [(1000, 128, 3001), (77, 4, 5), (5000, 64, 2500), (300, 200, 1237),
                                          (4096, 512, 700)])
def test_row_table_pull_push_match_torch(rows, width, n):
    """Keyed pull (with snapshot) and the add / scaled_add / max / assign pushes of a row table
    against plain PyTorch indexing in fp64; ids repeat, so pushes to one row accumulate."""
    from paracel_b200.ps.tables import RowTable
    g = torch.Generator(device="cuda").manual_seed(rows + width)
    t = RowTable(rows, width)
    ref = torch.randn(rows, width, device="cuda", generator=g)
    t.shard[:rows] = ref
    ids = torch.randint(0, rows, (n,), device="cuda", generator=g)
    out = torch.empty(n, width, device="cuda")
    snap = torch.empty(n, width, device="cuda")
    t.pull(ids, out, snap)
    t.check()
    assert torch.equal(out, ref[ids]) and torch.equal(snap, ref[ids])
    # add with per-row weights: table += w * (cur - old); old is refreshed to cur
    cur = out + torch.randn(n, width, device="cuda", generator=g)
    w = torch.rand(n, device="cuda", generator=g)
    exp = ref.double().index_add_(0, ids, (cur - snap).double() * w.double()[:, None])
    t.push(ids, cur, snap, w, handler="add", start=n // 3)
    t.check()
    assert (t.shard[:rows].double() - exp).abs().max().item() < 1e-4
    assert torch.equal(snap, cur)
    # scaled add without snapshot: table += scale * cur
    exp = t.shard[:rows].double().index_add_(0, ids, 0.25 * cur.double())
    t.push(ids, cur, None, None, handler="scaled_add", scale=0.25)
    t.check()
    assert (t.shard[:rows].double() - exp).abs().max().item() < 1e-4
    # max
    before = t.shard[:rows].clone()
    exp = before.clone().index_reduce_(0, ids, cur, "amax", include_self=True)
    t.push(ids, cur, None, None, handler="max")
    t.check()
    assert torch.equal(t.shard[:rows], exp)
    # assign on distinct ids
    uids = torch.randperm(rows, device="cuda", generator=g)[: min(rows, n)]
    vals = torch.randn(uids.numel(), width, device="cuda", generator=g)
    t.push(uids, vals, None, None, handler="assign")
    t.check()
    assert torch.equal(t.shard[:rows][uids], vals)
    t.free()


def test_running_topk_and_gram():
    from paracel_b200.ops.misc import RunningTopK, gram
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(9)
    m, n, k = 300, 1000, 7
    S = torch.randn(m, n, device=dev, generator=g)
    row_ids = torch.arange(m, device=dev) * 3
    col_ids = torch.arange(n, device=dev)
    tk = RunningTopK(row_ids, k, lower=0.5)
    for c0 in range(0, n, 256):           # tiles arrive one after the other
        tk.update(S[:, c0:c0 + 256].contiguous(), col_ids[c0:c0 + 256])
    torch.cuda.synchronize()
    res = tk.result()
    Sm = S.clone()
    Sm[row_ids[:, None] == col_ids[None, :]] = -1e30   # self excluded
    for r in (0, 1, 150, 299):
        vals, idx = torch.topk(Sm[r], k)
        exp = [(int(i), float(v)) for v, i in zip(vals, idx) if v >= 0.5]
        got = res.get(int(row_ids[r]), [])
        assert [i for i, _ in got] == [i for i, _ in exp]
        assert np.allclose([v for _, v in got], [v for _, v in exp])
    H = torch.randn(5000, 50, device=dev, generator=g)
    G = gram(H)
    torch.cuda.synchronize()
    torch.testing.assert_close(G.double(), H.double().T @ H.double(), rtol=1e-4, atol=1e-2)


def test_device_allreduce_single_rank():
    from paracel_b200.ops.misc import DeviceAllReduce
    ar = DeviceAllReduce(device="cuda:0")
    x = torch.arange(10, dtype=torch.float64, device="cuda:0")
    for _ in range(3):
        y = ar(x)
    torch.cuda.synchronize()
    ar.check()
    assert torch.equal(x, y)
    ar.free()


def test_device_balltree_search_matches_host_tree_and_brute_force():
    import numpy as np
    from paracel_b200.tool.balltree import DeviceBalltree, PyBalltree, PyQuery, balltree_search_with_dp
    rng = np.random.default_rng(4)
    items = rng.standard_normal((6000, 24)) * rng.uniform(0.2, 2.0, (6000, 1))
    tree = PyBalltree(items)
    tree.build()
    dt = DeviceBalltree(tree)
    queries = rng.standard_normal((300, 24))
    k = 7
    idx, sc, vis = dt.search(queries, k)
    torch.cuda.synchronize()
    idx, sc, vis = idx.cpu().numpy(), sc.cpu().numpy(), vis.cpu().numpy()
    exact = (queries @ items.T)
    ref_idx = np.argsort(-exact, axis=1)[:, :k]
    ref_sc = np.take_along_axis(exact, ref_idx, axis=1)
    assert np.allclose(sc, ref_sc, rtol=1e-4, atol=1e-4)          # same scores as brute force
    assert (idx == ref_idx).mean() > 0.995                          # ids differ only on fp32 near-ties
    assert np.all(np.diff(sc, axis=1) <= 1e-6)                      # best first
    assert vis.min() > 0 and vis.max() < tree.node_count            # some balls were pruned
    host = balltree_search_with_dp(PyQuery(list(queries[0]), k), tree)
    assert [i for i, _ in host] == list(idx[0])
    assert abs(tree.last_visited - int(vis[0])) <= 0.05 * tree.last_visited   # same traversal
    # fewer items than k
    small = PyBalltree(items[:3])
    small.build()
    i2, s2, _ = DeviceBalltree(small).search(queries[:2], 5)
    assert (i2[:, 3:] == -1).all().item() and sorted(i2[0, :3].tolist()) == [0, 1, 2]
