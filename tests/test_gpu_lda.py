"""GPU collapsed-Gibbs LDA: count bookkeeping is exact and the sampler mixes like the serial
CPU sampler (log-likelihood curves agree statistically)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _corpus(ndocs=300, V=400, topics=4, doc_len=60, seed=0):
    rng = np.random.default_rng(seed)
    phi = rng.dirichlet(np.full(V, 0.02), topics)
    ptr, words = [0], []
    for d in range(ndocs):
        theta = rng.dirichlet(np.full(topics, 0.2))
        n = int(rng.poisson(doc_len)) + 1
        zz = rng.choice(topics, n, p=theta)
        words.extend(int(rng.choice(V, p=phi[t])) for t in zz)
        ptr.append(len(words))
    return np.asarray(ptr, dtype=np.int64), np.asarray(words, dtype=np.int64)


def test_lda_gpu_counts_and_likelihood():
    from paracel_b200._core import core
    from paracel_b200.models.lda_gpu import LdaGibbsGpu
    ptr, words = _corpus()
    V, K, alpha, beta, iters = 400, 128, 0.1, 0.05, 25
    m = LdaGibbsGpu(V, K, alpha, beta, iters=iters, nbatch=3, staleness=0, device="cuda:0", seed=1)
    m.load_docs(torch.tensor(ptr), torch.tensor(words))
    T = len(words)
    assert int(m.wt.shard.sum().item()) == T and int(m.ts.shard.sum().item()) == T
    ll = m.fit(with_loglik=True)
    torch.cuda.synchronize()
    # bookkeeping stays exact: every token is counted once in every table
    assert int(m.wt.shard.sum().item()) == T and int(m.ts.shard.sum().item()) == T
    assert int(m.n_dk.sum().item()) == T
    assert torch.equal(m.n_dk.sum(1).int(), m.doc_len)
    assert torch.equal(m.wt.shard[:V].sum(0).int(), m.ts.shard[0].int())
    zc = torch.bincount(m.z.long(), minlength=K).int()
    assert torch.equal(zc, m.ts.shard[0].int())
    assert int(m.wt.shard.min().item()) >= 0
    # serial CPU sampler on the same corpus
    rng = np.random.default_rng(1)
    lens = np.diff(ptr).astype(np.int32)
    z = rng.integers(0, K, size=T, dtype=np.int32)
    nd = np.zeros((len(lens), K), dtype=np.int32)
    np.add.at(nd, (np.repeat(np.arange(len(lens)), lens), z), 1)
    nw = np.zeros((V, K), dtype=np.int32)
    np.add.at(nw, (words, z), 1)
    nk = np.bincount(z, minlength=K).astype(np.int32)
    w32 = words.astype(np.int32)
    ll_cpu = []
    for it in range(iters):
        core().lda_gibbs_sweep(ptr, w32, z, nd, nw, nk, lens, K, V, alpha, beta, 100 + it)
        theta = (nd + alpha) / (lens[:, None] + K * alpha)
        phi = (nw + beta) / (nk[None, :] + V * beta)
        doc_of = np.repeat(np.arange(len(lens)), lens)
        ll_cpu.append(float(np.log((theta[doc_of] * phi[words]).sum(1)).sum()))
    assert ll[-1] > ll[0] + 0.05 * abs(ll[0])
    assert abs(ll[-1] - ll_cpu[-1]) < 0.03 * abs(ll_cpu[-1]), (ll[-1], ll_cpu[-1])
    assert m.perplexity(ll[-1]) < V
    m.free()


@pytest.mark.parametrize("K", [256, 1024])
def test_lda_gpu_other_topic_counts(K):
    from paracel_b200.models.lda_gpu import LdaGibbsGpu
    ptr, words = _corpus(ndocs=120, V=200, doc_len=40, seed=2)
    m = LdaGibbsGpu(200, K, iters=4, nbatch=2, staleness=0, device="cuda:0")
    m.load_docs(torch.tensor(ptr), torch.tensor(words))
    ll = m.fit(with_loglik=True)
    torch.cuda.synchronize()
    T = len(words)
    assert int(m.wt.shard.sum().item()) == T and int(m.n_dk.sum().item()) == T
    assert torch.equal(torch.bincount(m.z.long(), minlength=K).int(), m.ts.shard[0].int())
    assert ll[-1] > ll[0]
    m.free()
