"""Checkpoint / resume of the device models: N steps in one go against N/2 steps, save, a fresh
object, load, N/2 steps.  PageRank and dense logistic regression have no atomics whose order
could differ: they must agree exactly (dense LR: to fp32 rounding of its block reduction).
LDA and k-means restore their sampler / centre state."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_pagerank_resume_is_exact(tmp_path):
    from paracel_b200.models.pagerank_gpu import PageRankGpu
    g = torch.Generator(device=DEV).manual_seed(1)
    n, m = 5000, 60000
    src = torch.randint(0, n, (m,), device=DEV, generator=g)
    dst = torch.randint(0, n, (m,), device=DEV, generator=g)

    def make():
        pr = PageRankGpu(n, 0.85, device=DEV)
        pr.load_edges(src, dst)
        return pr
    a = make()
    a.run(7)                      # an odd count: the ping-pong tables swap roles across the save
    full = a.ranks().clone()
    a.free()
    b = make()
    b.run(3)
    b.save_checkpoint(str(tmp_path / "ck"))
    b.free()
    c = make()
    c.load_checkpoint(str(tmp_path / "ck"))
    assert c.it == 3
    c.run(4)
    # the edge-balanced kernel joins the partial sums of a row that spans blocks with atomics, whose
    # order may differ between launches: equal to fp32 rounding, not necessarily bit for bit
    torch.testing.assert_close(c.ranks(), full, rtol=2e-6, atol=1e-9)
    c.free()


def test_dense_lr_resume(tmp_path):
    from paracel_b200.models.linear_gpu import DenseLinearGpu
    g = torch.Generator().manual_seed(2)
    n, d = 4000, 33
    X = torch.randn(n, d, generator=g)
    y = (torch.rand(n, generator=g) < 0.5).float()
    th0 = torch.rand(d, generator=g)

    def make():
        m = DenseLinearGpu(d, eta=0.5, device=DEV)
        m.load(X, y, theta0=th0.to(DEV))
        return m
    a = make()
    for _ in range(8):
        a.step()
    full = a.weights()
    a.free()
    b = make()
    for _ in range(4):
        b.step()
    b.save_checkpoint(str(tmp_path / "ck"))
    b.free()
    c = make()
    c.load_checkpoint(str(tmp_path / "ck"))
    for _ in range(4):
        c.step()
    torch.testing.assert_close(c.weights(), full, rtol=1e-5, atol=1e-6)
    c.free()


def test_lda_and_kmeans_resume(tmp_path):
    from paracel_b200.models.kmeans_gpu import KMeansGpu
    from paracel_b200.models.lda_gpu import LdaGibbsGpu
    rng = np.random.default_rng(3)
    V, K, ndocs = 200, 128, 150
    ptr, words = [0], []
    for _ in range(ndocs):
        words.extend(rng.integers(0, V, int(rng.integers(20, 50))).tolist())
        ptr.append(len(words))
    ptr, words = torch.tensor(ptr), torch.tensor(words)

    def make_lda():
        m = LdaGibbsGpu(V, K, iters=8, nbatch=2, staleness=0, device=DEV, seed=5)
        m.load_docs(ptr, words)
        return m
    a = make_lda()
    ll_full = a.fit(with_loglik=True)
    a.free()
    b = make_lda()
    for _ in range(4):
        b.iteration()
    b.save_checkpoint(str(tmp_path / "lda"))
    b.free()
    c = make_lda()
    c.load_checkpoint(str(tmp_path / "lda"))
    assert c.step_no == 8 and c.clock == 8
    T = int(words.numel())
    assert int(c.wt.shard.sum().item()) == T and int(c.n_dk.sum().item()) == T
    ll_rest = c.fit(with_loglik=True)
    assert len(ll_rest) == 4
    # same seeds per step and one warp per document: the resumed sampler continues the same chain
    assert abs(ll_rest[-1] - ll_full[-1]) < 0.02 * abs(ll_full[-1])
    assert int(c.wt.shard.sum().item()) == T
    c.free()
    # k-means: centres after 3 + 3 rounds equal 6 rounds
    g = torch.Generator(device=DEV).manual_seed(6)
    X = torch.randn(3000, 5, device=DEV, generator=g) + 4 * torch.randint(0, 3, (3000, 1), device=DEV, generator=g)

    def make_km():
        m = KMeansGpu(6, 5, device=DEV)
        m.load(X, init_centres=X[:6].clone())
        return m
    a = make_km()
    a.fit(6)
    full = a.cluster_centres()
    a.free()
    b = make_km()
    b.fit(3)
    b.save_checkpoint(str(tmp_path / "km"))
    b.free()
    c = make_km()
    c.load_checkpoint(str(tmp_path / "km"))
    c.fit(3)
    torch.testing.assert_close(c.cluster_centres(), full, rtol=1e-5, atol=1e-5)
    c.free()
