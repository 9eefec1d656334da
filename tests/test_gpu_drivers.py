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


def test_pagerank_driver_matches_power_iteration(monkeypatch, tmp_path):
    from paracel_b200.utils import dump as D
    edges = [(10, 20), (10, 30), (20, 30), (30, 10), (40, 30), (40, 10), (50, 40)]
    inp = tmp_path / "pr.txt"
    inp.write_text("".join(f"{a},{b}\n" for a, b in edges) + "60,2147483648\n")
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
    assert abs(miu["rating_sz"] - 20000) < 0.5 and 2.5 < miu["miu"] < 3.5

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
