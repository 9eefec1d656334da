"""Multi-GPU tests (2 ranks, one process per GPU, NCCL for plumbing and plain
peer loads/stores in the kernels).  NVLS is switched off for these runs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs2 = pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")


def _job(n):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from paracel_b200.launch.local import LocalJob
    return LocalJob(n, 0, backend="cpu:gloo,cuda:nccl")


@needs2
def test_symmetric_buffers_and_row_tables_across_ranks():
    from workers.gpu_workers import symm_and_rows
    res = _job(2).run(symm_and_rows, timeout_s=300)
    for r in res:
        assert r["peer_vals"] == [1.0, 2.0]
        assert r["pull_ok"] and r["push_ok"] and r["int_ok"]


@needs2
def test_device_ssp_clock_bound_and_timeout():
    from workers.gpu_workers import ssp_clock
    res = _job(2).run(ssp_clock, timeout_s=300)
    assert res[0]["max_ahead"] <= 2
    assert res[0]["timeout"] not in (None, "none")
    assert res[0]["alive"] == 4.0


@needs2
def test_mf_two_ranks_converges_like_one_rank():
    from workers.gpu_workers import mf_train
    args = (3000, 800, 200_000, 32, 5, 2)
    two = _job(2).run(mf_train, args, timeout_s=300)
    one = _job(1).run(mf_train, args, timeout_s=300)
    assert two[0]["nnz_local"] + two[1]["nnz_local"] == 200_000
    assert abs(two[0]["rmse1"] - two[1]["rmse1"]) < 1e-6  # all-reduced metric
    assert two[0]["rmse1"] < two[0]["rmse0"]
    assert abs(two[0]["rmse1"] - one[0]["rmse1"]) < 0.05 * one[0]["rmse1"]


@needs2
@pytest.mark.parametrize("kernel", ["1sm", "2sm", "2sm-wide"])
def test_fused_allgather_gemm_two_ranks(kernel):
    from workers.gpu_workers import fused_gather_gemm
    res = _job(2).run(fused_gather_gemm, (1000, 64, 900, kernel), timeout_s=300)
    for r in res:
        assert r["err0"] < 5e-3 and r["err1"] < 5e-3, r
        assert r["argmin_ok"]


@needs2
def test_dense_table_reduce_scatter_handler_two_ranks():
    from workers.gpu_workers import dense_table_two_ranks
    assert all(_job(2).run(dense_table_two_ranks, timeout_s=300))


@needs2
def test_sparse_l1lr_and_pagerank_two_ranks():
    from workers.gpu_workers import l1lr_and_pagerank_two_ranks
    for ok_lr, ok_pr in _job(2).run(l1lr_and_pagerank_two_ranks, timeout_s=300):
        assert ok_lr and ok_pr


@needs2
def test_kmeans_allreduce_lda_two_ranks():
    from workers.gpu_workers import kmeans_allreduce_lda_two_ranks
    for r in _job(2).run(kmeans_allreduce_lda_two_ranks, timeout_s=300):
        assert r["allreduce"] and r["kmeans"], r
        assert r["lda_counts"][0] == r["lda_counts"][2] == r["lda_counts"][1], r
        assert r["lda_ll_up"] and r["lda_consistent"], r


@needs2
@pytest.mark.parametrize("pattern", ["fmap", "fsmap"])
def test_device_loader_exchange_two_ranks(pattern):
    from workers.gpu_workers import device_exchange_ranks
    res = _job(2).run(device_exchange_ranks, (pattern,), timeout_s=300)
    assert sum(r["n"] for r in res) == 100_000
    for r in res:
        assert r["triples"] and r["maps"] and r["idx"], r


@needs2
def test_paralg_api_on_device_tables_two_ranks():
    from workers.gpu_workers import paralg_device_backend_two_ranks
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from paracel_b200.launch.local import LocalJob
    for r in LocalJob(2, 1, backend="cpu:gloo,cuda:nccl").run(paralg_device_backend_two_ranks, timeout_s=300):
        assert r == {"row_read": True, "row_in_owner_hbm": True, "dense_equals_host": True,
                     "batch_push": True, "filter_view": True}, r


@needs2
def test_first_read_of_a_collectively_written_key_waits_for_every_owner():
    from workers.gpu_workers import dense_linear_first_read_sees_theta0
    assert all(_job(2).run(dense_linear_first_read_sees_theta0, timeout_s=300))


@needs2
def test_als_svd_similarity_mvv_two_ranks():
    from workers.gpu_workers import suite_models_two_ranks
    for r in _job(2).run(suite_models_two_ranks, timeout_s=600):
        assert r["als"] and r["svd_sigma"] and r["svd_recon"] and r["sim_dense"] and r["mvv"], r


@needs2
def test_launcher_gpu_switch_runs_pagerank_on_two_gpus(tmp_path):
    """prun --gpu: two workers, one GPU each, reference input in and pagerank_0 out."""
    import json
    import random
    import subprocess
    import sys
    random.seed(1)
    edges = [(random.randrange(1, 300), random.randrange(1, 300)) for _ in range(4000)]
    inp = tmp_path / "edges.txt"
    inp.write_text("".join(f"{a},{b}\n" for a, b in edges))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps({"input": str(inp), "output": str(tmp_path / "out") + "/", "rounds": 6,
                               "damping_factor": 0.85}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root,
               PARACEL_RUN_LOG=str(tmp_path / "paracelrun_log"))
    rc = subprocess.run([sys.executable, "-m", "paracel_b200.launch.prun", "-w", "2", "-p", "1", "-c", str(cfg),
                         "-m", "local", "--gpu", "pagerank"], env=env, cwd=root, timeout=300).returncode
    assert rc == 0
    got = {}
    for line in open(tmp_path / "out" / "pagerank_0"):
        k, v = line.split("\t")
        got[int(k)] = float(v)
    srcs = sorted({a for a, _ in edges})
    assert sorted(got) == srcs
    # power iteration in plain Python over the distinct edges: a repeated input line is one edge,
    # as in the host path, whose graph container keeps adj[v][w]
    edges = sorted(set(edges))
    nodes = sorted({a for a, _ in edges} | {b for _, b in edges})
    outdeg = {v: 0 for v in nodes}
    for a, _ in edges:
        outdeg[a] += 1
    n_out = sum(1 for v in nodes if outdeg[v] > 0)
    pr = {v: (1.0 / n_out if outdeg[v] > 0 else 0.0) for v in nodes}
    for _ in range(6):
        nxt = {v: 0.15 for v in nodes}
        for a, b in edges:
            nxt[b] += 0.85 * pr[a] / outdeg[a]
        pr = nxt
    for v in srcs[:50]:
        assert abs(got[v] - pr[v]) < 1e-3 * max(1.0, pr[v])


def _prun_gpu(tmp_path, workers, algorithm, cfg, tag):
    """Run one device driver through the launcher with ``workers`` GPUs; returns the output dir."""
    import json
    import subprocess
    import sys
    out = tmp_path / f"{algorithm}_{tag}"
    cfg = dict(cfg, output=str(out) + ("/" if algorithm != "gLDA" else "_"))
    p = tmp_path / f"{algorithm}_{tag}.json"
    p.write_text(json.dumps(cfg))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root,
               PARACEL_RUN_LOG=str(tmp_path / "paracelrun_log"))
    rc = subprocess.run([sys.executable, "-m", "paracel_b200.launch.prun", "-w", str(workers), "-p", "1", "-c",
                         str(p), "-m", "local", "--gpu", algorithm], env=env, cwd=root, timeout=600).returncode
    assert rc == 0, (algorithm, workers)
    return out


def _read_all(outdir, prefix, reader):
    """Union of the per-rank dump files ``prefix<rank>`` of a run."""
    import glob
    merged = {}
    for f in sorted(glob.glob(os.path.join(str(outdir), prefix + "*"))):
        merged.update(reader(f))
    return merged


@needs2
def test_device_drivers_give_the_same_dumps_on_one_and_two_gpus(tmp_path):
    """Partitioned loading (every rank parses its byte range, ids are numbered jointly, entries
    travel to their owners) must not change what the drivers compute: ALS, max-vertex-value and
    dense similarity are deterministic and must agree between 1 and 2 workers; for MF the data
    summary (miu_0) and the key sets must."""
    import numpy as np
    from paracel_b200.utils import dump as D
    rng = np.random.default_rng(11)
    # ---- ALS
    nu, ni, k = 80, 50, 8
    H = rng.normal(size=(ni, k))
    fac = tmp_path / "H.txt"
    fac.write_text("".join("%d\t%s\n" % (700 + j, "|".join("%.6f" % v for v in H[j])) for j in range(ni)))
    pairs = sorted({(int(rng.integers(0, nu)), int(rng.integers(0, ni))) for _ in range(1500)})
    rat = tmp_path / "rating.txt"
    rat.write_text("".join("%d,%d,%.3f\n" % (100 + u, 700 + i, rng.uniform(1, 5)) for u, i in pairs))
    cfg = {"rating_input": str(rat), "factor_input": str(fac), "lambda": 0.2}
    one = _read_all(_prun_gpu(tmp_path, 1, "als", cfg, "w1"), "W_", D.read_dict_vector)
    two = _read_all(_prun_gpu(tmp_path, 2, "als", cfg, "w2"), "W_", D.read_dict_vector)
    assert set(one) == set(two) and len(one) == len({u for u, _ in pairs})
    for key in one:
        assert np.allclose(one[key], two[key], rtol=1e-4, atol=1e-4)
    # ---- max vertex value
    es, ed = rng.integers(1, 90, 260), rng.integers(1, 90, 260)
    mv = tmp_path / "mvv.txt"
    mv.write_text("".join("%d,%d\n" % (a, b) for a, b in zip(es, ed)))
    one = _read_all(_prun_gpu(tmp_path, 1, "mvv", {"input": str(mv)}, "w1"), "vertex_val_", D.read_dict_scalar)
    two = _read_all(_prun_gpu(tmp_path, 2, "mvv", {"input": str(mv)}, "w2"), "vertex_val_", D.read_dict_scalar)
    assert one == two and len(one) == len(set(es.tolist()))
    # ---- dense similarity
    N, d = 120, 10
    Xs = rng.normal(size=(N, d))
    si = tmp_path / "sim.txt"
    si.write_text("".join("%d,%s\n" % (2000 + j, ",".join("%.6f" % v for v in Xs[j])) for j in range(N)))
    cfg = {"input": str(si), "topk": 3, "simbar": -1.0}

    def lines(outdir):
        import glob
        out = []
        for f in glob.glob(os.path.join(str(outdir), "result_*")):
            out.extend(open(f).read().splitlines())
        return {l.split("\t")[0]: [p.split(":")[0] for p in l.split("\t")[1].split("|") if p] for l in out}
    one, two = lines(_prun_gpu(tmp_path, 1, "sim_dense", cfg, "w1")), lines(_prun_gpu(tmp_path, 2, "sim_dense", cfg, "w2"))
    assert one == two and len(one) == N
    # ---- MF: same data summary and key sets; repeated (user, item) lines on different ranks collapse
    lines_mf = []
    for _ in range(6000):
        u, i = int(rng.integers(0, 150)), int(rng.integers(0, 60))
        lines_mf.append(f"{10 + u} {500 + i} 2005-01-01 {int(rng.integers(1, 6))}\n")
    mf = tmp_path / "mf.txt"
    mf.write_text("".join(lines_mf))
    cfg = {"input": str(mf), "k": 16, "rounds": 3, "alpha": 0.01, "beta": 0.02}
    o1, o2 = _prun_gpu(tmp_path, 1, "mf", cfg, "w1"), _prun_gpu(tmp_path, 2, "mf", cfg, "w2")
    m1, m2 = D.read_dict_scalar(str(o1 / "miu_0")), D.read_dict_scalar(str(o2 / "miu_0"))
    assert m1["rating_sz"] == m2["rating_sz"] == len({tuple(l.split()[:2]) for l in lines_mf})
    assert abs(m1["miu"] - m2["miu"]) < 1e-5
    assert set(D.read_dict_vector(str(o1 / "W_0"))) == set(D.read_dict_vector(str(o2 / "W_0")))
    assert set(D.read_dict_scalar(str(o1 / "ibias_0"))) == set(D.read_dict_scalar(str(o2 / "ibias_0")))
