"""The launcher-facing GPU drivers: reference input files in, reference dump files out."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(monkeypatch, tmp_path, algorithm, cfg):
    from paracel_b200 import run
    monkeypatch.setenv("PCL_USE_GPU", "1")
    p = tmp_path / f"{algorithm}.json"
    p.write_text(json.dumps(cfg))
    assert run.main([algorithm, "--server_info", "", "--cfg_file", str(p)]) == 0


def _run_cpu(monkeypatch, tmp_path, algorithm, cfg):
    """The host driver of the same executable, against parameter servers in this process."""
    from paracel_b200 import run
    from paracel_b200.ps.server import LocalServers
    monkeypatch.setenv("PCL_USE_GPU", "0")
    p = tmp_path / f"{algorithm}_cpu.json"
    p.write_text(json.dumps(cfg))
    with LocalServers(1) as srv:
        assert run.main([algorithm, "--server_info", srv.info(), "--cfg_file", str(p)]) == 0


def test_pagerank_driver_matches_power_iteration(monkeypatch, tmp_path):
    from paracel_b200.utils import dump as D
    edges = [(10, 20), (10, 30), (20, 30), (30, 10), (40, 30), (40, 10), (50, 40)]
    inp = tmp_path / "pr.txt"
    # a repeated line is still one edge (the containers of the reference keep adj[v][w])
    inp.write_text("".join(f"{a},{b}\n" for a, b in edges) + "60,2147483648\n" + "10,20\n40,30\n")
    out = tmp_path / "pr_out"
    _run(monkeypatch, tmp_path, "pagerank", {"input": str(inp), "output": str(out) + "/", "rounds": 12,
                                              "damping_factor": 0.85})
    nodes = [10, 20, 30, 40, 50, 60]
    outdeg = {v: sum(1 for a, _ in edges if a == v) for v in nodes}
    outdeg[60] = 1
    pr = {v: 1.0 / 6 for v in nodes}
    for _ in range(12):
        pr = {v: 0.15 + 0.85 * sum(pr[a] / outdeg[a] for a, b in edges if b == v) for v in nodes}
    got = D.read_dict_scalar(os.path.join(str(out), "pagerank_0"))
    assert set(got) == {str(v) for v in nodes}
    for v in nodes:
        assert abs(got[str(v)] - pr[v]) < 1e-4
    # and the host driver writes the same file for the same input
    out_cpu = tmp_path / "pr_cpu"
    _run_cpu(monkeypatch, tmp_path, "pagerank", {"input": str(inp), "output": str(out_cpu) + "/", "rounds": 12,
                                                  "damping_factor": 0.85})
    cpu = D.read_dict_scalar(os.path.join(str(out_cpu), "pagerank_0"))
    assert set(cpu) == set(got)
    for v in cpu:
        assert abs(cpu[v] - got[v]) < 1e-4


def test_kmeans_and_lr_drivers(monkeypatch, tmp_path):
    from paracel_b200.utils import dump as D
    rng = np.random.default_rng(0)
    X = np.concatenate([rng.normal(0, 0.3, (60, 4)), rng.normal(5, 0.3, (60, 4))])
    order = rng.permutation(120)
    order = np.concatenate([[0, 60], order[(order != 0) & (order != 60)]])   # one seed per blob first
    inp = tmp_path / "km.txt"
    inp.write_text("".join("%d\t%s\n" % (i, ",".join("%.6f" % v for v in X[i])) for i in order))
    out = tmp_path / "km_out"
    _run(monkeypatch, tmp_path, "kmeans", {"input": str(inp), "output": str(out) + "/", "kclusters": 2,
                                            "rounds": 5})
    groups = [l.rstrip("\n").split("\t")[1].split("|") for l in open(out / "kmeans_0")]
    assert sorted(len(g) for g in groups) == [60, 60]
    centres = D.read_dict_vector(os.path.join(str(out), "centers_0"))
    firsts = sorted(v[0] for v in centres.values())
    assert abs(firsts[0] - X[:60, 0].mean()) < 1e-3 and abs(firsts[1] - X[60:, 0].mean()) < 1e-3

    n, d = 4000, 8
    A = rng.standard_normal((n, d))
    w = rng.standard_normal(d)
    y = (rng.random(n) < 1 / (1 + np.exp(-A @ w))).astype(float)
    tr = tmp_path / "lr.csv"
    np.savetxt(tr, np.concatenate([A, y[:, None]], 1), delimiter=",", fmt="%.6f")
    lo = tmp_path / "lr_out"
    _run(monkeypatch, tmp_path, "lr", {"training_input": str(tr), "output": str(lo) + "/", "rounds": 200,
                                        "alpha": 0.0005, "beta": 0.0})
    theta = np.asarray([float(x) for x in open(lo / "lr_theta_0").read().strip().split("|")])
    assert theta.shape == (d + 1,)
    assert np.corrcoef(theta[1:], w)[0, 1] > 0.95        # the weights point the right way


def test_mf_and_lda_drivers(monkeypatch, tmp_path):
    from paracel_b200.utils import dump as D
    rng = np.random.default_rng(1)
    nu, ni = 300, 120
    P, Q = rng.normal(0, 0.5, (nu, 4)), rng.normal(0, 0.5, (ni, 4))
    lines = []
    for _ in range(20000):
        u, i = rng.integers(0, nu), rng.integers(0, ni)
        r = int(np.clip(np.rint(3 + P[u] @ Q[i] + rng.normal(0, 0.3)), 1, 5))
        lines.append(f"{1000 + u} {5000 + i} 2005-01-01 {r}\n")
    inp = tmp_path / "mf.txt"
    inp.write_text("".join(lines))
    out = tmp_path / "mf_out"
    _run(monkeypatch, tmp_path, "mf", {"input": str(inp), "output": str(out) + "/", "k": 16, "rounds": 30,
                                        "alpha": 0.01, "beta": 0.02})
    W = D.read_dict_vector(os.path.join(str(out), "W_0"))
    H = D.read_dict_vector(os.path.join(str(out), "H_0"))
    assert len(W) == nu and len(H) == ni and all(1000 <= int(k) < 1000 + nu for k in W)
    assert len(next(iter(W.values()))) == 16
    miu = D.read_dict_scalar(os.path.join(str(out), "miu_0"))
    # a repeated (user, item) line replaces the earlier rating, as in the host path
    last = {}
    for l in lines:
        f = l.split()
        last[(f[0], f[1])] = float(f[3])
    assert abs(miu["rating_sz"] - len(last)) < 0.5
    assert abs(miu["miu"] - sum(last.values()) / len(last)) < 1e-4

    vocab_a, vocab_b = [f"a{j}" for j in range(30)], [f"b{j}" for j in range(30)]
    docs = []
    for dno in range(200):
        v = vocab_a if dno % 2 == 0 else vocab_b
        docs.append(" ".join(rng.choice(v, 40)) + "\n")
    li = tmp_path / "lda.txt"
    li.write_text("".join(docs))
    lo = tmp_path / "lda_out_"
    _run(monkeypatch, tmp_path, "gLDA", {"input": str(li), "output": str(lo), "k_topics": 128, "iters": 30,
                                          "alpha": 0.1, "beta": 0.01, "top_words": 5})
    rows = [l.rstrip("\n") for l in open(str(lo) + "0")]
    assert len(rows) == 128 and rows[0].startswith("0topic\t") and rows[0].endswith("|")
    # a topic's top words come from one of the two disjoint vocabularies
    pure = 0
    for r in rows:
        ws = [x.split(":")[0] for x in r.split("\t")[1].split("|") if x]
        pure += len({w[0] for w in ws}) == 1
    assert pure > 80      # (nearly empty topics list arbitrary words)


def test_ridge_and_l1_drivers(monkeypatch, tmp_path):
    rng = np.random.default_rng(2)
    n, d = 3000, 6
    A = rng.standard_normal((n, d))
    w = rng.standard_normal(d)
    yv = A @ w + 0.7 + 0.01 * rng.standard_normal(n)
    tr = tmp_path / "ridge.csv"
    np.savetxt(tr, np.concatenate([A, yv[:, None]], 1), delimiter=",", fmt="%.6f")
    out = tmp_path / "ridge_out"
    _run(monkeypatch, tmp_path, "ridge", {"training_input": str(tr), "output": str(out) + "/", "rounds": 60,
                                           "alpha": 0.001, "beta": 0.0, "method": "ipm"})
    theta = np.asarray([float(x) for x in open(out / "ridge_theta_0").read().strip().split("|")])
    assert np.allclose(theta[1:], w, atol=0.05) and abs(theta[0] - 0.7) < 0.05
    # sparse L1 logistic regression: the informative features survive, most others are zero
    n, d = 6000, 40
    X = (rng.random((n, d)) < 0.15).astype(float)
    wt = np.zeros(d)
    wt[:4] = [3.0, -3.0, 2.5, -2.5]
    y = (rng.random(n) < 1 / (1 + np.exp(-(X @ wt)))).astype(float)
    inp = tmp_path / "l1.csv"
    np.savetxt(inp, np.concatenate([X, y[:, None]], 1), delimiter=",", fmt="%.1f")
    out = tmp_path / "l1_out"
    _run(monkeypatch, tmp_path, "lr_l1", {"input": str(inp), "output": str(out) + "/", "rounds": 300,
                                           "eta": 2.0, "lambda": 60.0})   # 0.01 per sample
    wv = np.asarray([float(x) for x in open(out / "lr_l1_weight_0").read().strip().split("|")])
    assert wv.shape == (d,)
    assert np.all(np.sign(wv[:4]) == np.sign(wt[:4])) and np.all(np.abs(wv[:4]) > 0.5)
    assert (wv[4:] == 0).sum() >= 30


def test_als_svd_sim_mvv_drivers_match_the_host_drivers(monkeypatch, tmp_path):
    from paracel_b200.utils import dump as D
    rng = np.random.default_rng(3)
    # ---- ALS
    nu, ni, k = 60, 40, 8
    H = rng.normal(size=(ni, k))
    fac = tmp_path / "H.txt"
    fac.write_text("".join("%d\t%s\n" % (500 + j, "|".join("%.6f" % v for v in H[j])) for j in range(ni)))
    pairs = {(int(rng.integers(0, nu)), int(rng.integers(0, ni))) for _ in range(900)}
    rat = tmp_path / "rating.txt"
    rat.write_text("".join("%d,%d,%.3f\n" % (100 + u, 500 + i, rng.uniform(1, 5)) for u, i in sorted(pairs)))
    cfg = {"rating_input": str(rat), "factor_input": str(fac), "lambda": 0.2}
    _run(monkeypatch, tmp_path, "als", dict(cfg, output=str(tmp_path / "als_gpu") + "/"))
    _run_cpu(monkeypatch, tmp_path, "als", dict(cfg, output=str(tmp_path / "als_cpu") + "/"))
    g = D.read_dict_vector(str(tmp_path / "als_gpu" / "W_0"))
    c = D.read_dict_vector(str(tmp_path / "als_cpu" / "W_0"))
    assert set(g) == set(c) and len(g) > 50
    for key in c:
        assert np.allclose(g[key], c[key], rtol=2e-3, atol=2e-3)
    # ---- SVD
    m, n = 80, 30
    M = (rng.normal(size=(m, 3)) * np.array([8.0, 5.0, 3.0])) @ rng.normal(size=(3, n))
    sv = tmp_path / "svd.txt"
    sv.write_text("".join("%d,%d,%.6f\n" % (r, cc, M[r, cc]) for r in range(m) for cc in range(n)))
    cfg = {"input": str(sv), "k": 3}
    _run(monkeypatch, tmp_path, "svd", dict(cfg, output=str(tmp_path / "svd_gpu") + "/"))
    sg = np.asarray([float(x) for x in open(tmp_path / "svd_gpu" / "SIGMA_0").read().replace("\n", ",").strip(",").split(",")])
    assert np.allclose(sg, np.linalg.svd(M, compute_uv=False)[:3], rtol=2e-3)
    U = D.read_dict_vector(str(tmp_path / "svd_gpu" / "U_0"))
    V = D.read_dict_vector(str(tmp_path / "svd_gpu" / "V_0"))
    rec = np.asarray([U[str(r)] for r in range(m)]) * sg[None, :] @ np.asarray([V[str(cc)] for cc in range(n)]).T
    assert np.abs(rec - M).max() < 1e-2 * np.abs(M).max()
    # ---- dense similarity
    N, d = 90, 12
    Xs = rng.normal(size=(N, d))
    si = tmp_path / "sim.txt"
    si.write_text("".join("%d,%s\n" % (1000 + j, ",".join("%.6f" % v for v in Xs[j])) for j in range(N)))
    cfg = {"input": str(si), "topk": 4, "simbar": -1.0}
    _run(monkeypatch, tmp_path, "sim_dense", dict(cfg, output=str(tmp_path / "sim_gpu") + "/"))
    _run_cpu(monkeypatch, tmp_path, "sim_dense", dict(cfg, output=str(tmp_path / "sim_cpu") + "/"))
    gl = sorted(open(tmp_path / "sim_gpu" / "result_0").read().splitlines())
    cl = sorted(open(tmp_path / "sim_cpu" / "result_0").read().splitlines())
    assert len(gl) == N == len(cl)

    def parse(lines):
        out = {}
        for l in lines:
            key, rest = l.split("\t")
            out[key] = [(p.split(":")[0], float(p.split(":")[1])) for p in rest.split("|") if p]
        return out
    pg, pc = parse(gl), parse(cl)
    for key in pc:
        assert [a for a, _ in pg[key]] == [a for a, _ in pc[key]]
        assert np.allclose([b for _, b in pg[key]], [b for _, b in pc[key]], atol=1e-4)
    # ---- max vertex value
    es, ed = rng.integers(1, 60, 150), rng.integers(1, 60, 150)
    mv = tmp_path / "mvv.txt"
    mv.write_text("".join("%d,%d\n" % (a, b) for a, b in zip(es, ed)))
    cfg = {"input": str(mv)}
    _run(monkeypatch, tmp_path, "mvv", dict(cfg, output=str(tmp_path / "mvv_gpu") + "/"))
    _run_cpu(monkeypatch, tmp_path, "mvv", dict(cfg, output=str(tmp_path / "mvv_cpu") + "/"))
    vg = D.read_dict_scalar(str(tmp_path / "mvv_gpu" / "vertex_val_0"))
    vc = D.read_dict_scalar(str(tmp_path / "mvv_cpu" / "vertex_val_0"))
    assert vg == vc and len(vg) > 20
