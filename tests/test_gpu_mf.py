"""GPU tests of the sparse row pull/push kernels, the device SSP clock and the
MF-SGD pass, each against a plain PyTorch / Python fp64 oracle."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _seq_mf_pass(u, i, r, W, H, bu, bi, mu, alpha, beta):
    """Sequential fp64 pass in the given order (mf.hpp:266-280)."""
    W, H, bu, bi = W.double().clone(), H.double().clone(), bu.double().clone(), bi.double().clone()
    for uu, ii, rr in zip(u.tolist(), i.tolist(), r.tolist()):
        pred = mu + bu[uu] + bi[ii] + (W[uu] * H[ii]).sum()
        pred = min(5.0, max(1.0, float(pred)))
        e = rr - pred
        dW = alpha * (2 * e * H[ii] - beta * W[uu])
        dH = alpha * (2 * e * W[uu] - beta * H[ii])
        W[uu] += dW
        H[ii] += dH
        bu[uu] += alpha * (2 * e - beta * bu[uu])
        bi[ii] += alpha * (2 * e - beta * bi[ii])
    return W, H, bu, bi


def test_rows_pull_push_match_index_ops():
    from paracel_b200.ps.tables import RowTable, ScalarTable
    dev = "cuda:0"
    torch.manual_seed(0)
    for width in (4, 8, 128, 132):
        t = RowTable(1000, width, torch.float32, device=dev)
        t.shard.copy_(torch.randn_like(t.shard))
        ref = t.shard.clone()
        ids = torch.randint(0, 1000, (777,), device=dev)
        ids = torch.unique(ids)
        cur = torch.empty(ids.numel(), width, device=dev)
        old = torch.empty_like(cur)
        t.pull(ids, cur, old)
        torch.cuda.synchronize()
        assert torch.equal(cur, ref[ids]) and torch.equal(old, ref[ids])
        delta = torch.randn_like(cur)
        cur += delta
        wgt = torch.rand(ids.numel(), device=dev)
        t.push(ids, cur, old, wgt)
        torch.cuda.synchronize()
        exp = ref.clone()
        exp[ids] += wgt[:, None] * delta
        torch.testing.assert_close(t.shard, exp, rtol=1e-5, atol=1e-5)
        assert torch.equal(old, cur)  # snapshot refreshed
        # duplicate ids accumulate
        dup = torch.tensor([3, 3, 3, 5], device=dev)
        ones = torch.ones(4, width, device=dev)
        before = t.shard.clone()
        t.push(dup, ones)
        torch.cuda.synchronize()
        assert torch.allclose(t.shard[3], before[3] + 3) and torch.allclose(t.shard[5], before[5] + 1)
        # max handler
        big = torch.full((1, width), 1e6, device=dev)
        t.push(torch.tensor([7], device=dev), big, handler="max")
        neg = torch.full((1, width), -1e6, device=dev)
        t.push(torch.tensor([8], device=dev), neg, handler="max")
        torch.cuda.synchronize()
        assert torch.all(t.shard[7] == 1e6)
        assert torch.equal(t.shard[8], before[8])
        t.free()
    s = ScalarTable(500, device=dev)
    ids = torch.arange(0, 500, 3, device=dev)
    v = torch.randn(ids.numel(), device=dev)
    s.push(ids, v)
    out = torch.empty_like(v)
    s.pull(ids, out)
    torch.cuda.synchronize()
    torch.testing.assert_close(out, v)
    s.free()


def test_rows_int32():
    from paracel_b200.ps.tables import RowTable
    dev = "cuda:0"
    t = RowTable(300, 1024, torch.int32, device=dev)
    ids = torch.tensor([1, 5, 299], device=dev)
    cur = torch.zeros(3, 1024, dtype=torch.int32, device=dev)
    old = torch.zeros_like(cur)
    t.pull(ids, cur, old)
    cur += torch.arange(1024, device=dev, dtype=torch.int32)[None, :] - 512
    t.push(ids, cur, old)
    t.push(ids, cur - old + torch.ones_like(cur))  # old == cur after refresh -> adds ones
    torch.cuda.synchronize()
    exp = torch.arange(1024, device=dev, dtype=torch.int32) - 512 + 1
    assert torch.equal(t.shard[5], exp) and torch.equal(t.shard[299], exp)
    assert int(t.shard[2].abs().sum()) == 0
    t.free()


def test_ssp_clock_commit_wait_and_timeout():
    from paracel_b200.parallel.ssp_device import DeviceSspClock, SspTimeout, DEPARTED
    c = DeviceSspClock(staleness=1, total_iters=3, device="cuda:0", timeout_s=0.05)
    c.wait()
    c.check()
    c.commit()
    c.commit()
    torch.cuda.synchronize()
    assert int(c.clocks[0]) == 2
    c.wait()
    c.check()
    # a flag that nothing sets: the wait must give up and report, not hang
    c.clock = 10
    c.wait()
    with pytest.raises(SspTimeout) as ei:
        c.check()
    assert ei.value.expected == 9 and ei.value.seen == 2
    c.clock = 2
    c.commit()  # reaches total_iters: departs
    torch.cuda.synchronize()
    assert int(c.clocks[0]) == DEPARTED
    c.free()


def test_mf_single_chunk_matches_sequential_oracle():
    from paracel_b200.models.mf_gpu import MfSgdGpu
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    # host: ratings streamed from pinned host memory (at rank 128 in the three-byte form)
    for k, hot, variant, compact, host in (
            (32, 64, 0, True, False), (80, 64, 0, False, False), (128, 64, 1, True, False),
            (128, 0, 1, False, False), (64, 3, 0, True, False), (128, 64, 2, True, False),
            (100, 0, 2, True, False), (128, 4, 2, True, False), (128, 64, 3, True, False),
            (128, 0, 3, False, False), (100, 4, 3, True, False), (128, 5, 3, False, False),
            (128, 64, 0, True, True), (128, 0, 3, True, True), (100, 4, 0, True, True)):
        nu, ni, nnz = 6, 9, 31
        u = torch.randint(0, nu, (nnz,), generator=g)
        i = torch.randint(0, ni, (nnz,), generator=g)
        r = torch.randint(1, 6, (nnz,), generator=g).float()
        m = MfSgdGpu(nu, ni, k=k, alpha=0.05, beta=0.02, rounds=1, device=dev, hot_rows=hot,
                     variant=variant, compact=compact)
        m.load_ratings(u, i, r, keep_on_host=host)
        m.init_parameters()
        assert torch.all(m.su == 1) and torch.all(m.si == 1)
        if host:
            assert m.packed_bits == 24 and m.h_packed.numel() == 24 * m.nchunks
        W0 = m.Wt.shard[:nu, :k].cpu()
        H0 = m.Ht.shard[:ni, :k].cpu()
        bu0, bi0 = m.but.shard[:nu].cpu(), m.bit.shard[:ni].cpu()
        order = torch.argsort(u, stable=True)
        We, He, bue, bie = _seq_mf_pass(u[order], i[order], r[order], W0, H0, bu0, bi0, m.mu,
                                        0.05, 0.02)
        m.round()
        torch.cuda.synchronize()
        lu, li = m.lu.cpu(), m.li.cpu()
        torch.testing.assert_close(m.Wt.shard[:nu, :k].cpu()[lu].double(), We[lu], rtol=2e-4, atol=2e-5)
        torch.testing.assert_close(m.Ht.shard[:ni, :k].cpu()[li].double(), He[li], rtol=2e-4, atol=2e-5)
        torch.testing.assert_close(m.but.shard[:nu].cpu()[lu].double(), bue[lu], rtol=2e-4, atol=2e-5)
        torch.testing.assert_close(m.bit.shard[:ni].cpu()[li].double(), bie[li], rtol=2e-4, atol=2e-5)
        if k < m.D:
            assert float(m.Wt.shard[:, k:].abs().sum()) == 0.0
        m.free()


def test_round_result_handles():
    """round() returns a handle to the pass's squared error: it agrees with the device-side sum
    when read at once, stays readable while later rounds are queued, and refuses to answer once
    its slot has been reused."""
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.synth import MfRatingStream
    dev = "cuda:0"
    st = MfRatingStream(1500, 400, 20_000, seed=3, device=dev)
    u, i, r = st.chunk_at(0)
    m = MfSgdGpu(1500, 400, k=32, rounds=12, device=dev, staleness=0, ssp=False)
    m.load_ratings(u, i, r)
    m.init_parameters()
    first = m.round()
    assert first.sse() == float(m.sse.item()) and first.sse() > 0
    held = [m.round() for _ in range(3)]             # three rounds queued, none read yet
    vals = [h.sse() for h in held]
    assert all(v > 0 for v in vals) and vals[0] != vals[1]
    assert vals[-1] == float(m.sse.item())
    assert vals[-1] < first.sse()                    # the error of the pass goes down
    old = m.round()
    for _ in range(MfSgdGpu.RESULT_SLOTS):
        m.round()
    with pytest.raises(RuntimeError):
        old.sse()
    assert first.sse() > 0                           # a value that was read stays available
    m.paracel_check()
    m.free()


def test_mf_converges_like_sequential_pass():
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.synth import MfRatingStream
    dev = "cuda:0"
    _converges(32)
    _converges(128)
    _converges(128, variant=1)


def _converges(k, variant=0):
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.synth import MfRatingStream
    dev = "cuda:0"
    nu, ni, nnz = 2000, 600, 30_000
    st = MfRatingStream(nu, ni, nnz, seed=5, device=dev)
    u, i, r = st.chunk_at(0)
    rounds = 4
    m = MfSgdGpu(nu, ni, k=k, alpha=0.005, beta=0.02, rounds=rounds, device=dev, staleness=0,
                 ssp=False, variant=variant)
    m.load_ratings(u, i, r)
    m.init_parameters()
    m.pull()
    r0 = m.rmse()
    W0 = m.Wt.shard[:nu, :k].cpu()
    H0 = m.Ht.shard[:ni, :k].cpu()
    bu0, bi0 = m.but.shard[:nu].cpu(), m.bit.shard[:ni].cpu()
    m.fit()
    r_gpu = m.rmse()
    # vectorised fp64 oracle: sequential pass in user-major order
    order = torch.argsort(u.cpu(), stable=True)
    uu, ii, rr = u.cpu()[order], i.cpu()[order], r.cpu()[order]
    W, H, bu, bi = W0, H0, bu0, bi0
    for _ in range(rounds):
        W, H, bu, bi = _seq_mf_pass(uu[:], ii[:], rr[:], W, H, bu, bi, m.mu, 0.005, 0.02)
    pred = (m.mu + bu[uu] + bi[ii] + (W[uu] * H[ii]).sum(1)).clamp(1, 5)
    r_cpu = math.sqrt(float(((rr.double() - pred) ** 2).mean()))
    pr = m.predict(u[:100], i[:100]).cpu()
    assert torch.all((pr >= 1) & (pr <= 5))
    m.free()
    assert r_gpu < r0
    assert abs(r_gpu - r_cpu) < 0.10 * r_cpu, (r0, r_gpu, r_cpu)


def test_mf_streamed_rounds_equal_resident_rounds_statistically():
    from paracel_b200.models.mf_gpu import MfSgdGpu
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(11)
    nu, ni, nnz = 500, 300, 60_000
    u = torch.randint(0, nu, (nnz,), device=dev, generator=g)
    i = torch.randint(0, ni, (nnz,), device=dev, generator=g)
    r = torch.randint(1, 6, (nnz,), device=dev, generator=g).float()
    out = []
    for host, compact in ((False, True), (True, True), (True, False)):
        m = MfSgdGpu(nu, ni, k=64, rounds=4, device=dev, seed=1, compact=compact)
        m.load_ratings(u, i, r, keep_on_host=host)
        m.init_parameters()
        m.fit()
        out.append(m.rmse())
        if host:
            assert m.h2d_bytes == ((m.packed_bits * 4 + 12) if compact else 12 * 32) * m.nchunks
        m.free()
    assert abs(out[0] - out[1]) < 0.02 * out[0] and abs(out[0] - out[2]) < 0.02 * out[0], out


def test_mf_heldout_rmse_tracks_the_sequential_pass_on_zipf_ratings():
    """Where the kernel's approximations are active -- hot item rows replicated per CTA and
    averaged, concurrency weights below one -- the held-out RMSE after 1, 2, 5 and 10 epochs
    stays within a stated distance of the fp64 sequential pass over the ratings in shuffled
    order (1.15 / 1.12 / 1.08 / 1.06 times its RMSE), and below the sequential pass in the
    order the reference visits ratings (user by user, mf.hpp:313 over its bigraph), at every
    epoch.  Zipf(1.1) ids, 50 k x 10 k, 5 M ratings, rank 128, 5 % held out."""
    import numpy as np
    from paracel_b200._core import core
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.synth import MfRatingStream
    dev = torch.device("cuda:0")
    nu, ni, nnz, k, epochs = 50_000, 10_000, 5_000_000, 128, 10
    u, i, r = MfRatingStream(nu, ni, nnz, s=1.1, seed=1, device=dev).chunk_at(0)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    perm = torch.randperm(nnz, device=dev, generator=g)
    nh = nnz // 20
    hu, hi, hr = u[perm[:nh]], i[perm[:nh]], r[perm[:nh]]
    tu, ti, tr = u[perm[nh:]], i[perm[nh:]], r[perm[nh:]]
    marks = (1, 2, 5, 10)
    m = MfSgdGpu(nu, ni, k=k, alpha=0.005, beta=0.02, rounds=epochs, staleness=0, ssp=False, device=dev, seed=3)
    m.load_ratings(tu, ti, tr)
    m.init_parameters()
    assert m.hot_T > 0 and float(m.su.min()) < 1.0          # the approximations are in play
    W0 = m.Wt.shard[:nu, :k].double().cpu().numpy().copy()
    H0 = m.Ht.shard[:ni, :k].double().cpu().numpy().copy()
    bu0, bi0 = m.but.shard[:nu].double().cpu().numpy().copy(), m.bit.shard[:ni].double().cpu().numpy().copy()
    mu = m.mu
    gpu = {}
    for e in range(1, epochs + 1):
        m.round()
        if e in marks:
            sse, cnt = m.heldout_sse(hu, hi, hr)
            gpu[e] = math.sqrt(sse / cnt)
    m.paracel_check()
    m.free()
    hu_c, hi_c, hr_c = hu.cpu().numpy(), hi.cpu().numpy(), hr.double().cpu().numpy()

    def sequential(order):
        uu = np.ascontiguousarray(tu.cpu().numpy().astype(np.int64)[order])
        ii = np.ascontiguousarray(ti.cpu().numpy().astype(np.int64)[order])
        rr = np.ascontiguousarray(tr.double().cpu().numpy()[order])
        W, H, bu, bi = W0.copy(), H0.copy(), bu0.copy(), bi0.copy()
        out = {}
        for e in range(1, epochs + 1):
            core().mf_sgd_pass(uu, ii, rr, W, H, bu, bi, mu, 0.005, 0.02)
            if e in marks:
                p = np.clip(mu + bu[hu_c] + bi[hi_c] + (W[hu_c] * H[hi_c]).sum(1), 1, 5)
                out[e] = float(np.sqrt(((p - hr_c) ** 2).mean()))
        return out
    n_train = nnz - nh
    shuffled = sequential(np.arange(n_train))                 # the split above is a random permutation
    user_rank = np.random.default_rng(0).permutation(nu)
    by_user = sequential(np.argsort(user_rank[tu.cpu().numpy()], kind="stable"))
    tol = {1: 1.15, 2: 1.12, 5: 1.08, 10: 1.06}
    for e in marks:
        assert gpu[e] <= tol[e] * shuffled[e], (e, gpu, shuffled)
        assert gpu[e] < by_user[e], (e, gpu, by_user)
    assert gpu[10] < gpu[5] < gpu[2] < gpu[1]


def test_mf_checkpoint_resume_and_metrics(tmp_path):
    """N rounds in one go against N/2 rounds, checkpoint, a fresh object, load, N/2 rounds: the
    held-in RMSE agrees within 1 % (the kernel's atomics reorder, so not bit for bit); the
    run writes one metrics line per round and a phase trace."""
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.metrics import MetricsLogger
    from paracel_b200.utils.synth import MfRatingStream
    dev = "cuda:0"
    nu, ni, nnz, N = 3000, 800, 200_000, 6
    u, i, r = MfRatingStream(nu, ni, nnz, seed=9, device=dev).chunk_at(0)

    def make(rounds_done=0):
        m = MfSgdGpu(nu, ni, k=32, rounds=N, staleness=0, ssp=False, device=dev, seed=4,
                     output=str(tmp_path / "out"))
        m.load_ratings(u, i, r)
        m.init_parameters()
        return m
    a = make()
    a.paracel_enable_metrics(str(tmp_path / "metrics.jsonl"))
    a.metrics_sync = True
    a.fit()
    full = a.rmse()
    a.dump_phase_trace(str(tmp_path / "trace.json"))
    a.free()
    lines = MetricsLogger.read(str(tmp_path / "metrics.jsonl"))
    assert len(lines) == N and lines[-1]["round"] == N and lines[0]["ratings"] == nnz
    assert lines[0]["bytes_pulled"] > 0 and lines[-1]["sse_of_pass"] < lines[0]["sse_of_pass"]
    import json
    tr = json.load(open(tmp_path / "trace.json"))
    assert tr["phases"]["sgd"]["count"] == N and tr["phases"]["sgd"]["ms"] > 0
    b = make()
    for _ in range(N // 2):
        b.round()
    b.save_checkpoint(str(tmp_path / "ckpt"))
    b.free()
    c = make()
    c.load_checkpoint(str(tmp_path / "ckpt"))
    assert c.clock == N // 2
    c.fit()                                     # the remaining N / 2 rounds
    assert c.clock == N
    resumed = c.rmse()
    c.free()
    assert abs(resumed - full) < 0.01 * full, (resumed, full)
