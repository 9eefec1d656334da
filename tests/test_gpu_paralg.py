"""The paralg API on the device backend (one GPU): string keys and key batches resolve to
rows of HBM tables, handler names select the kernel's reduction, non-table keys still go to
the host servers, id range checks report instead of faulting."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pt(**kw):
    from paracel_b200.paralg import paralg
    from paracel_b200.ps.server import LocalServers
    srv = LocalServers(1)
    pt = paralg(srv.info(), backend="gpu", device="cuda:0", **kw)
    return pt, srv


def test_string_keys_reach_device_rows_and_host_keys_reach_the_server():
    pt, srv = _pt()
    try:
        names = np.array([3, 10, 123, 4000], dtype=np.int64)
        W = pt.paracel_row_table(4, 8, prefix="W_", names=names, handler="mf_fac_updater")
        B = pt.paracel_scalar_table(16, prefix="usr_bias_")
        pt.paracel_dense_table("theta", 10, handler="lr_theta_update")
        # write / read by string key
        pt.paracel_write("W_123", [1.0, 2.0, 3.0])
        pt.paracel_write("usr_bias_5", 0.25)
        pt.paracel_write("theta", torch.arange(10.0))
        pt.paracel_write("plain_key", {"a": 1})                  # host server
        pt.paracel_sync()
        row = pt.paracel_read("W_123")
        assert row.is_cuda and row.tolist() == [1.0, 2.0, 3.0, 0, 0, 0, 0, 0]
        assert W.table.shard[2].tolist() == row.tolist()         # names[2] == 123, one rank: row 2
        assert pt.paracel_read("usr_bias_5") == 0.25
        assert pt.paracel_read("theta").tolist() == list(range(10))
        assert pt.paracel_read("plain_key") == {"a": 1}
        assert pt.paracel_contains("W_10") and not pt.paracel_contains("W_11")
        with pytest.raises(KeyError):
            pt.paracel_read("W_11")                              # not a row of the table, not on the host
        # bupdate with handler names
        pt.paracel_bupdate("W_123", [1.0] * 8, "", "mf_fac_updater")
        pt.paracel_bupdate("usr_bias_5", 0.5, "", "mf_bias_updater")
        pt.paracel_bupdate("usr_bias_5", 0.1, "", "max_updater")
        pt.paracel_bupdate("usr_bias_6", -2.0, "", "max_updater")
        pt.paracel_bupdate("theta", torch.ones(10), "", "lr_theta_update")                    # one-sided add
        pt.paracel_bupdate("theta", torch.ones(10), "", "lr_theta_update", collective=True)   # reduce-scatter
        pt.paracel_bupdate("theta", torch.full((10,), 4.0), "", "sgd", lr=0.25)               # theta -= 1
        pt.paracel_sync()
        assert pt.paracel_read("W_123").tolist() == [2.0, 3.0, 4.0, 1, 1, 1, 1, 1]
        assert pt.paracel_read("usr_bias_5") == 0.75
        assert pt.paracel_read("usr_bias_6") == 0.0               # max(0, -2)
        assert pt.paracel_read("theta").tolist() == [x + 1.0 for x in range(10)]
        # multi forms on strings: mixed device and host keys
        pt.paracel_write_multi({"W_3": [9.0] * 8, "usr_bias_1": 1.5, "other": 7})
        pt.paracel_bupdate_multi(["usr_bias_1", "usr_bias_2"], [0.5, 2.0], "", "mf_bias_updater")
        pt.paracel_sync()
        got = pt.paracel_read_multi(["usr_bias_1", "W_3", "other", "usr_bias_2"])
        assert got[0] == 2.0 and got[1].tolist() == [9.0] * 8 and got[2] == 7 and got[3] == 2.0
        # filters see device tables by their key pattern
        d = pt.paracel_read_special("", "mf_W_filter")
        assert set(d) == {"W_3", "W_10", "W_123", "W_4000"} and d["W_3"] == [9.0] * 8
        ub = pt.paracel_read_special("", "mf_ubias_filter")
        assert len(ub) == 16 and ub["usr_bias_5"] == 0.75
        assert "plain_key" in pt.paracel_readall() and "theta" in pt.paracel_readall()
        # prox-L1 is not linear: only the collective form exists
        with pytest.raises(ValueError):
            pt.paracel_bupdate("theta", torch.ones(10), "", "prox_l1", collective=False)
        pt.paracel_check()
    finally:
        pt.close()
        srv.stop()


def test_key_batches_pull_push_and_update_future():
    pt, srv = _pt()
    try:
        T = pt.paracel_row_table(1000, 128, prefix="H_")
        T.table.shard.copy_(torch.arange(1000.0, device="cuda")[:, None].expand(1000, 128))
        ids = torch.tensor([5, 999, 17, 5], device="cuda")
        kb = pt.paracel_keys(T, ids)
        assert kb.keys() == ["H_5", "H_999", "H_17", "H_5"]
        out = torch.empty(4, 128, device="cuda")
        snap = torch.empty_like(out)
        pt.paracel_read_multi(kb, out=out, snapshot=snap)
        assert out[:, 0].tolist() == [5.0, 999.0, 17.0, 5.0] and torch.equal(out, snap)
        out += 1.0
        w = torch.tensor([1.0, 0.5, 1.0, 1.0], device="cuda")
        pt.paracel_bupdate_multi(kb, out, "", "mf_fac_updater", old=snap, wgt=w)
        fut = pt.paracel_update("H_17", [10.0] * 128, "", "default_incr_lf")
        assert fut.result() is True and fut.done()
        pt.paracel_sync()
        assert float(T.table.shard[5, 3]) == 7.0          # two holders of row 5 added 1 each
        assert float(T.table.shard[999, 0]) == 999.5
        assert float(T.table.shard[17, 127]) == 28.0
        assert torch.equal(out, snap)                      # snapshot refreshed by the push
        pt.paracel_check()
    finally:
        pt.close()
        srv.stop()


def test_out_of_range_ids_are_reported_and_skipped():
    from paracel_b200.ops._lib import BadDeviceId, validate_ids
    pt, srv = _pt()
    try:
        T = pt.paracel_row_table(100, 8, prefix="R_")
        T.table.shard.fill_(1.0)
        # the allocation is rounded up and owned by this process: even a missed check could not
        # leave it; the check must skip the row and report it
        ids = torch.tensor([3, 100, 7], device="cuda")
        out = torch.full((3, 8), -5.0, device="cuda")
        T.table.pull(ids, out)
        torch.cuda.synchronize()
        assert out[0].tolist() == [1.0] * 8 and out[2].tolist() == [1.0] * 8
        assert out[1].tolist() == [-5.0] * 8               # untouched
        with pytest.raises(BadDeviceId) as e:
            pt.paracel_check()
        assert e.value.bad_id == 100 and e.value.position == 1
        T.table.push(torch.tensor([-1, 2], device="cuda"), torch.ones(2, 8, device="cuda"))
        with pytest.raises(BadDeviceId) as e:
            pt.paracel_check()
        assert e.value.bad_id == -1
        assert float(T.table.shard.sum()) == 100 * 8 + 8   # only row 2 changed
        # a push that finds an error in its status block does nothing
        st = torch.zeros(4, dtype=torch.int64, device="cuda")
        st[0] = 1
        T.table.push(torch.tensor([4], device="cuda"), torch.ones(1, 8, device="cuda"), status=st)
        torch.cuda.synchronize()
        assert float(T.table.shard[4].sum()) == 8.0
        with pytest.raises(BadDeviceId):
            validate_ids(torch.tensor([0, 5, 12], dtype=torch.int32, device="cuda"), 0, 12, "test ids")
        validate_ids(torch.tensor([0, 5, -1], dtype=torch.int32, device="cuda"), 0, 12, "test ids", skip=-1)
    finally:
        pt.close()
        srv.stop()


def test_device_models_are_paralg_subclasses():
    from paracel_b200.models.kmeans_gpu import KMeansGpu
    from paracel_b200.models.lda_gpu import LdaGibbsGpu
    from paracel_b200.models.linear_gpu import DenseLinearGpu, SparseLinearGpu
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.models.pagerank_gpu import PageRankGpu
    from paracel_b200.paralg import paralg
    for cls in (MfSgdGpu, SparseLinearGpu, DenseLinearGpu, LdaGibbsGpu, PageRankGpu, KMeansGpu):
        assert issubclass(cls, paralg)
    m = MfSgdGpu(50, 20, k=32, rounds=2, device="cuda:0")
    u = torch.randint(0, 50, (500,), device="cuda")
    i = torch.randint(0, 20, (500,), device="cuda")
    m.load_ratings(u, i, torch.randint(1, 6, (500,), device="cuda").float())
    m.solve()
    row = m.paracel_read("W_7")                # the public key of a factor row
    assert torch.equal(row, m.Wt.shard[7])
    d = m.paracel_read_special("", "mf_H_filter")
    assert len(d) == 20 and d["H_3"] == m.Ht.shard[3].tolist()
    m.free()


def test_clock_commit_is_withheld_after_a_failed_wait():
    """A rank whose staleness wait ran out must not announce progress: the commit kernel looks
    at the status block on the device and stores nothing while it holds an error."""
    from paracel_b200.parallel.ssp_device import DeviceSspClock, SspTimeout
    c = DeviceSspClock(1, 10, device="cuda:0")
    c.commit()
    torch.cuda.synchronize()
    assert int(c.clocks[0]) == 1
    c.status[0] = 1                    # what a timed-out wait leaves behind
    c.commit()
    torch.cuda.synchronize()
    assert int(c.clocks[0]) == 1       # not announced
    with pytest.raises(SspTimeout):
        c.check()                      # reports and clears
    c.commit()
    torch.cuda.synchronize()
    assert int(c.clocks[0]) == 3
    c.free()


def test_ssp_cache_rule_on_device_reads():
    """Under SSP a copy pulled at clock c is served while clock - c < limit_s (no kernel runs),
    the first read and the reads after the last iteration always pull."""
    from paracel_b200.ops import _lib
    from paracel_b200.paralg import paralg
    pt = paralg(None, rounds=6, limit_s=2, ssp_switch=True, backend="gpu", device="cuda:0")
    try:
        T = pt.paracel_row_table(64, 8, prefix="R_")
        pt.paracel_dense_table("theta", 40)
        kb = pt.paracel_keys(T, torch.arange(0, 64, 3, device="cuda"))
        out = torch.empty(len(kb), 8, device="cuda")
        pulls = []
        for it in range(6):
            n0 = _lib.launches()
            pt.paracel_read_multi(kb, out=out)
            pt.paracel_read("theta")
            pulls.append(_lib.launches() - n0)
            pt.paracel_bupdate_multi(kb, torch.ones(len(kb), 8, device="cuda"), "", "add")
            pt.iter_commit()
        # clock 0: pull; 1: cached; 2: pull (2 clocks old); 3: cached; 4: pull; 5: cached
        assert [p > 0 for p in pulls] == [True, False, True, False, True, False]
        n0 = _lib.launches()
        pt.paracel_read_multi(kb, out=out)            # clock == total_iters: always pulls
        assert _lib.launches() > n0
        torch.cuda.synchronize()
        assert float(out[0, 0]) == 6.0                 # six pushes of one arrived at the owner
        assert pt.paracel_would_pull(kb, out)
        pt.paracel_check()
    finally:
        pt.close()


def test_vertex_programs_on_device_tables():
    """The vectorised Pregel layer: max-value propagation and min-plus shortest paths against
    plain Python fixpoints."""
    import numpy as np
    from paracel_b200.pregel_gpu import MaxValueVertices, ShortestPaths
    rng = np.random.default_rng(4)
    nv, ne = 300, 1200
    es, ed = rng.integers(0, nv, ne), rng.integers(0, nv, ne)
    w = rng.uniform(0.5, 2.0, ne).astype(np.float32)
    # shortest paths from vertex es[0]: Bellman-Ford oracle in float64
    src0 = int(es[0])
    dist = np.full(nv, np.inf)
    dist[src0] = 0.0
    for _ in range(nv):
        changed = False
        for a, b, ww in zip(es.tolist(), ed.tolist(), w.tolist()):
            if dist[a] + ww < dist[b] - 1e-12:
                dist[b] = dist[a] + ww
                changed = True
        if not changed:
            break
    sp = ShortestPaths(nv, src0, device="cuda:0")
    sp.load_edges(torch.tensor(es), torch.tensor(ed), torch.tensor(w))
    steps = sp.run_supersteps()
    got = sp.values_of(torch.arange(nv)).cpu().numpy()
    reach = np.isfinite(dist)
    assert steps > 1 and np.allclose(got[reach], dist[reach], rtol=1e-5, atol=1e-5)
    assert np.all(got[~reach] > 1e37)                  # unreachable vertices keep "infinity"
    sp.free()
    val = {int(v): float(v) for v in np.unique(es)}
    changed = True
    while changed:
        changed = False
        for a, b in zip(es.tolist(), ed.tolist()):
            if b in val and val[a] > val[b]:
                val[b] = val[a]
                changed = True
    mv = MaxValueVertices(nv, device="cuda:0")
    mv.load_edges(torch.tensor(es), torch.tensor(ed))
    mv.run_supersteps()
    assert dict(zip(mv.lv.cpu().tolist(), mv.val.cpu().tolist())) == val
    mv.free()
