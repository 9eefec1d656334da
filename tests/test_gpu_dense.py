"""Dense-table read / bupdate handlers, linear-model gradient kernels and the PageRank pull
step on one GPU, each against a PyTorch fp32/fp64 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_dense_table_handlers_single_rank():
    from paracel_b200.ps.tables import DenseTable
    dev = "cuda:0"
    L = 1003
    g = torch.Generator(device=dev).manual_seed(0)
    theta0 = torch.randn(L, device=dev, generator=g)
    for handler, lr, lam in (("add", 1.0, 0.0), ("sgd", 0.1, 0.0), ("prox_l1", 0.1, 0.5), ("max", 1.0, 0.0)):
        t = DenseTable(L, device=dev, handler=handler, lr=lr, lam=lam)
        t.write(theta0)
        torch.testing.assert_close(t.read(), theta0)
        exp = theta0.clone()
        for it in range(3):
            d = torch.randn(L, device=dev, generator=g)
            t.delta().copy_(d)
            t.bupdate(count_nnz=True)
            if handler == "add":
                exp = exp + d
            elif handler == "sgd":
                exp = exp - lr * d
            elif handler == "prox_l1":
                w = exp - lr * d
                exp = torch.sign(w) * torch.clamp(w.abs() - lr * lam, min=0)
            else:
                exp = torch.maximum(exp, d)
            got = t.read()
            torch.cuda.synchronize()
            t.check()
            torch.testing.assert_close(got, exp, rtol=1e-6, atol=1e-6)
            assert int(t.nnz.item()) == int((exp != 0).sum().item())
        t.free()


def test_dense_lr_gradient_matches_torch():
    from paracel_b200.ops.linear import DenseGrad
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(1)
    for n, d in ((5000, 101), (333, 7), (20000, 1024)):
        X = torch.randn(n, d, device=dev, generator=g)
        theta = 0.1 * torch.randn(d, device=dev, generator=g)
        y = (torch.rand(n, device=dev, generator=g) < 0.5).float()
        op = DenseGrad(d, dev)
        grad = torch.empty(d, device=dev)
        for _ in range(2):  # second call: the counter must have been left at zero
            loss = op(X, y, theta, grad, logistic=True)
            torch.cuda.synchronize()
            z = X.double() @ theta.double()
            h = torch.sigmoid(z)
            ref_g = X.double().T @ (y.double() - h)
            ref_loss = -(y.double() * torch.log(h) + (1 - y.double()) * torch.log(1 - h)).sum()
            torch.testing.assert_close(grad.double(), ref_g, rtol=2e-4, atol=2e-3)
            assert abs(float(loss.item()) - float(ref_loss)) < 1e-3 * abs(float(ref_loss))
        loss = op(X, y, theta, grad, logistic=False)
        torch.cuda.synchronize()
        r = y.double() - X.double() @ theta.double()
        torch.testing.assert_close(grad.double(), X.double().T @ r, rtol=2e-4, atol=2e-3)
        assert abs(float(loss.item()) - float((r * r).sum())) < 1e-3 * float((r * r).sum())


def test_sparse_lr_gradient_matches_torch():
    from paracel_b200.ops.linear import sparse_grad
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(2)
    n, F, nnz_row = 4000, 50000, 40
    cols = (torch.rand(n, nnz_row, device=dev, generator=g) ** 3 * F).long().clamp(max=F - 1)
    row_ptr = torch.arange(0, n * nnz_row + 1, nnz_row, device=dev, dtype=torch.int64)
    theta = 0.3 * torch.randn(F, device=dev, generator=g)
    y = (torch.rand(n, device=dev, generator=g) < 0.5).float()
    vals = torch.rand(n * nnz_row, device=dev, generator=g)
    for v in (None, vals):
        grad = torch.zeros(F, device=dev)
        loss = torch.zeros(1, device=dev, dtype=torch.float64)
        sparse_grad(row_ptr, cols.view(-1).int().contiguous(), v, y, theta, grad, loss, hot_T=4096)
        torch.cuda.synchronize()
        vv = torch.ones(n * nnz_row, device=dev, dtype=torch.float64) if v is None else v.double()
        z = (theta.double()[cols.view(-1)] * vv).view(n, nnz_row).sum(1)
        h = torch.sigmoid(z)
        r = y.double() - h
        ref = torch.zeros(F, device=dev, dtype=torch.float64)
        ref.index_add_(0, cols.view(-1), (r[:, None] * vv.view(n, nnz_row)).reshape(-1))
        torch.testing.assert_close(grad.double(), ref, rtol=1e-3, atol=1e-3)
        ref_loss = -(y.double() * torch.log(h) + (1 - y.double()) * torch.log(1 - h)).sum()
        assert abs(float(loss.item()) - float(ref_loss)) < 1e-3 * abs(float(ref_loss))


def test_pagerank_pull_matches_dense_reference():
    from paracel_b200.ops.linear import pagerank_pull
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(3)
    n, m = 3000, 40000
    src = torch.randint(0, n, (m,), device=dev, generator=g)
    dst = (torch.rand(m, device=dev, generator=g) ** 2 * n).long().clamp(max=n - 1)
    outdeg = torch.bincount(src, minlength=n).float()
    order = torch.argsort(dst, stable=True)
    cols = src[order].int().contiguous()
    row_ptr = torch.zeros(n + 1, device=dev, dtype=torch.int64)
    row_ptr[1:] = torch.cumsum(torch.bincount(dst, minlength=n), 0)
    inv = torch.where(outdeg > 0, 1.0 / outdeg.clamp(min=1), torch.zeros_like(outdeg))
    pr = torch.full((n,), 1.0 / n, device=dev)
    for tpr in (4, 8, 32):
        contrib = pr * inv
        newc = torch.empty(n, device=dev)
        newr = torch.empty(n, device=dev)
        dl = torch.zeros(1, device=dev, dtype=torch.float64)
        deg = row_ptr[1:] - row_ptr[:-1]
        heavy = torch.nonzero(deg > 40).flatten().int().contiguous() if tpr == 8 else None
        pagerank_pull(row_ptr, cols, contrib, inv, 0.85, newc, newr, dl, pr, threads_per_row=tpr,
                      heavy_rows=heavy, heavy_deg=40)
        torch.cuda.synchronize()
        ref = torch.zeros(n, device=dev, dtype=torch.float64)
        ref.index_add_(0, dst, contrib.double()[src])
        ref = 0.15 + 0.85 * ref
        torch.testing.assert_close(newr.double(), ref, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(newc, newr * inv, rtol=1e-6, atol=1e-8)
        tot = float((ref - pr.double()).abs().sum())
        assert abs(float(dl.item()) - tot) < 1e-5 * tot + 1e-6
    # edge-balanced variant: blocks own equal numbers of in-links, rows cut by block boundaries
    from paracel_b200.ops.linear import pagerank_pull_stream
    contrib = pr * inv
    acc = torch.full((n,), 7.0, device=dev)        # must be cleared by the call
    newc2 = torch.empty(n, device=dev)
    newr2 = torch.empty(n, device=dev)
    dl2 = torch.zeros(1, device=dev, dtype=torch.float64)
    pagerank_pull_stream(row_ptr, cols, contrib, inv, 0.85, acc, newc2, newr2, dl2, pr)
    torch.cuda.synchronize()
    torch.testing.assert_close(newr2.double(), ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(newc2, newr2 * inv, rtol=1e-6, atol=1e-8)
    assert abs(float(dl2.item()) - tot) < 1e-5 * tot + 1e-6


def _sparse_problem(dev, n=20000, F=4096, nnz_row=12, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    cols = (torch.rand(n, nnz_row, device=dev, generator=g) ** 2 * F).long().clamp(max=F - 1)
    w = torch.zeros(F, device=dev)
    idx = torch.randperm(F, device=dev, generator=g)[: F // 50]
    w[idx] = 2.0 * torch.randn(idx.numel(), device=dev, generator=g)
    z = w[cols].sum(1)
    y = (torch.rand(n, device=dev, generator=g) < torch.sigmoid(z)).float()
    row_ptr = torch.arange(0, n * nnz_row + 1, nnz_row, device=dev, dtype=torch.int64)
    return row_ptr, cols.view(-1).int().contiguous(), y, w


def test_sparse_l1_logistic_regression_single_gpu():
    from paracel_b200.models.linear_gpu import SparseLinearGpu, remap_by_frequency
    dev = "cuda:0"
    row_ptr, cols, y, w_true = _sparse_problem(dev)
    F = w_true.numel()
    cols2, order = remap_by_frequency(cols, F)
    m = SparseLinearGpu(F, eta=2.0, lam=2e-4, nbatch=4, device=dev, hot_T=1024)
    m.load(row_ptr, cols2, y)
    losses = []
    for ep in range(30):
        m.epoch()
        losses.append(m.mean_loss())
    torch.cuda.synchronize()
    m.table.check()
    w = m.weights()
    # oracle: the same proximal-gradient iteration in fp64 with plain torch ops
    th = torch.zeros(F, device=dev, dtype=torch.float64)
    n = y.numel()
    C = cols2.long().view(n, -1)
    b = torch.linspace(0, n, 5).long().tolist()
    for ep in range(30):
        for k in range(4):
            lo, hi = b[k], b[k + 1]
            z = th[C[lo:hi]].sum(1)
            r = y[lo:hi].double() - torch.sigmoid(z)
            g = torch.zeros(F, device=dev, dtype=torch.float64)
            g.index_add_(0, C[lo:hi].reshape(-1), r[:, None].expand(-1, C.shape[1]).reshape(-1))
            wv = th + (2.0 / (n / 4)) * g
            t = (2.0 / (n / 4)) * 2e-4
            th = torch.sign(wv) * torch.clamp(wv.abs() - t, min=0)
    torch.testing.assert_close(w.double(), th, rtol=2e-3, atol=2e-4)
    assert losses[-1] < losses[0]
    assert m.nnz_weights() == int((w != 0).sum().item()) <= F
    m.free()


def test_dense_logistic_regression_single_gpu():
    from paracel_b200.models.linear_gpu import DenseLinearGpu
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(4)
    n, d = 20000, 101
    X = torch.randn(n, d, device=dev, generator=g)
    X[:, 0] = 1.0
    w = torch.randn(d, device=dev, generator=g)
    y = (torch.rand(n, device=dev, generator=g) < torch.sigmoid(X @ w)).float()
    m = DenseLinearGpu(d, eta=1.0, device=dev)
    m.load(X, y)
    th = torch.zeros(d, device=dev, dtype=torch.float64)
    for it in range(40):
        m.step()
        h = torch.sigmoid(X.double() @ th)
        th = th + (1.0 / n) * (X.double().T @ (y.double() - h))
    torch.testing.assert_close(m.weights().double(), th, rtol=1e-3, atol=1e-4)
    assert m.mean_loss() < 0.45
    m.free()


def test_pagerank_gpu_matches_power_iteration():
    from paracel_b200.models.pagerank_gpu import PageRankGpu
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(6)
    n, m_edges = 5000, 60000
    src = torch.randint(0, n, (m_edges,), device=dev, generator=g)
    dst = (torch.rand(m_edges, device=dev, generator=g) ** 2 * n).long().clamp(max=n - 1)
    # one vertex that only has the "no out-link" marker
    src = torch.cat([src, torch.tensor([n - 1], device=dev)])
    dst = torch.cat([dst, torch.tensor([2147483648], device=dev)])
    pr = PageRankGpu(n, 0.85, device=dev)
    pr.load_edges(src, dst)
    pr.run(15)
    got = pr.ranks().double()
    outdeg = torch.bincount(src, minlength=n).double()
    has = outdeg > 0
    ref = torch.where(has, torch.full((n,), 1.0 / int(has.sum()), device=dev, dtype=torch.float64), torch.zeros(n, device=dev, dtype=torch.float64))
    real = dst != 2147483648
    s, d_ = src[real], dst[real]
    for _ in range(15):
        c = torch.where(has, ref / outdeg.clamp(min=1), torch.zeros_like(ref))
        acc = torch.zeros(n, device=dev, dtype=torch.float64)
        acc.index_add_(0, d_, c[s])
        ref = 0.15 + 0.85 * acc
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-6)
    pr.step(track_delta=True)
    assert float(pr.delta_l1.item()) >= 0.0
    pr.free()
