"""Multi-process CPU tests: gloo ranks plus host parameter-server daemons on 127.0.0.1
(the reference's local mode: `prun.py -w W -p P -m local`, .travis.yml:87-92).  Covers every
Comm primitive, the whole parameter-server operation table, SSP (bound, departure, timeout
by a withheld commit) and the algorithms end to end against NumPy oracles."""
import os

import numpy as np
import pytest

from paracel_b200.launch.local import LocalJob
from workers import cpu_workers as W
from paracel_b200.utils import dump as D


def test_comm_primitives_three_ranks():
    res = LocalJob(3, 0).run(W.comm_primitives, timeout_s=300)
    assert res[1]["p2p"] == [7, [1.5, 2.5], "hello", [("a", "b", 1.0), ("c", "d", 2.0)],
                             [[], [("x", "y", 3.0)]], {"k": [1, 2]}]
    for rk, r in enumerate(res):
        assert r["ring"] == {"from": (rk + 2) % 3}
        assert r["bcast"] == [0, "x"]
        assert r["bcastring"] == [0, 0, 1, 2, 10, 20]
        assert r["alltoall"] == [[s] * (rk + 1) for s in range(3)]
        assert r["alltoallring"] == [[s, rk] for s in range(3)]
        assert r["ar_int"] == 6 and r["ar_float"] == 1.5 and r["ar_list"] == [3.0, 3.0]
        assert r["ar_np"] == [3.0, 3.0, 3.0]
        assert r["split"][1:] == ((2, 2) if rk % 2 == 0 else (1, 1))
    assert res[0]["tree_sum"] == 6
    assert res[0]["tree_dict"] == {"n": 3, "0": 1, "1": 1, "2": 1}


def test_parameter_server_operation_table():
    res = LocalJob(2, 2).run(W.ps_ops, timeout_s=300)
    for r in res:
        assert r["read"] == [1.0, 2.0] and r["contains"] == (True, False)
        assert r["multi"] == [0, 1, 2, 3, 4] and r["multi_dict"] == {"m0_1": 1}
        assert r["missing"] == "KeyError"
        assert r["theta"] == [2.0, 2.0, 2.0]      # first update stores the delta, second adds
        assert r["prod"] == 4 and r["cnt"] == 2 and r["update_future"] is True
        assert r["bm"] == [4, 4, 4]
        assert r["special"] == ["bm0", "bm1", "bm2"] and r["special_py"] == ["k0", "k1"]
        assert r["topk"] == [("m0_4", 4), ("m0_3", 3)]
        assert r["after_remove"] == (False, False, True)


def test_ssp_bound_and_departure():
    res = LocalJob(2, 1).run(W.ssp_bound, (2, 8, 1, 0.03), timeout_s=300)
    assert res[0]["max_ahead"] <= 2 and res[1]["max_ahead"] <= 2
    assert res[0]["max_ahead"] >= 1          # the fast worker did run ahead
    assert res[0]["total"] == 16.0 and res[1]["total"] == 16.0
    # limit_s = 0 degenerates to lock step
    res = LocalJob(2, 1).run(W.ssp_bound, (0, 4, 0, 0.02), timeout_s=300)
    assert max(r["max_ahead"] for r in res) == 0


def test_ssp_withheld_commit_times_out_instead_of_hanging():
    res = LocalJob(2, 1).run(W.ssp_withheld_commit, timeout_s=120)
    assert res[0].startswith("timeout at clock")


def _lr_data(tmp_path, n=4000, d=20, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, d))
    w = rng.standard_normal(d)
    y = (rng.random(n) < 1 / (1 + np.exp(-X @ w))).astype(float)
    p = str(tmp_path / "train.csv")
    np.savetxt(p, np.concatenate([X, y[:, None]], 1), delimiter=",", fmt="%.6f")
    return p, X, y


def test_lr_two_workers_one_server_ssp(tmp_path):
    """Plumbing configuration: LR SGD, 2 workers + 1 server, SSP staleness 1, 10 rounds."""
    inp, X, y = _lr_data(tmp_path)
    out = str(tmp_path / "out")
    res = LocalJob(2, 1).run(W.run_lr, (inp, out, "ipm", True), timeout_s=300)
    assert res[0]["n"] + res[1]["n"] == 4000
    assert abs(res[0]["loss"] - res[1]["loss"]) < 1e-12
    # oracle: log-loss of the dumped theta computed with NumPy
    theta = np.array([float(x) for x in open(os.path.join(out, "lr_theta_0")).read().strip().split("|")])
    Xb = np.concatenate([np.ones((4000, 1)), np.round(X, 6)], 1)
    h = 1 / (1 + np.exp(-Xb @ theta))
    oracle = float(-(y * np.log(h) + (1 - y) * np.log(1 - h)).mean())
    assert abs(oracle - res[0]["loss"]) < 1e-4
    assert res[0]["loss"] < 0.45             # well below log 2 after 10 rounds
    preds = open(os.path.join(out, "pred_v_0")).read().strip().split("\n")
    assert len(preds) == res[0]["n"] and ":" in preds[0]


@pytest.mark.parametrize("method", ["dgd", "downpour", "agd"])
def test_lr_other_methods(tmp_path, method):
    inp, X, y = _lr_data(tmp_path, n=600 if method == "agd" else 2000, d=8)
    rounds = 2 if method == "agd" else 5
    res = LocalJob(2, 1).run(W.run_lr, (inp, str(tmp_path / "o"), method, False, rounds), timeout_s=300)
    assert res[0]["loss"] < 0.69 or method == "dgd"
    assert np.isfinite(res[0]["theta"]).all()


def test_word_count_two_workers_two_servers(tmp_path):
    text = ["the quick brown fox", "the lazy dog and the fox", "a dog-eared book_1 is not a dog"] * 40
    p = tmp_path / "wc.txt"
    p.write_text("\n".join(text) + "\n")
    for variant in ("learning", "learning_slow"):
        res = LocalJob(2, 2).run(W.run_wc, (str(p), 4, variant), timeout_s=300)
        assert res[0][:2] == [("the", 120), ("a", 80)] or res[0][:2] == [("the", 120), ("fox", 80)]
        assert dict(res[0])["the"] == 120
        assert res[0] == res[1]


def test_kmeans_two_blobs(tmp_path):
    rng = np.random.default_rng(0)
    X = np.concatenate([rng.normal(0, 0.3, (60, 3)), rng.normal(5, 0.3, (60, 3))])
    idx = rng.permutation(120)
    # the first two rows (the seeds) come from different blobs
    idx = np.concatenate([[0, 60], idx[(idx != 0) & (idx != 60)]])
    p = tmp_path / "km.txt"
    p.write_text("".join("%d\t%s\n" % (i, ",".join("%.6f" % v for v in X[i])) for i in idx))
    out = str(tmp_path / "km")
    res = LocalJob(2, 1).run(W.run_kmeans, (str(p), out, 2, 6), timeout_s=300)
    C = np.asarray(res[0]["clusters"])
    assert np.allclose(sorted(C[:, 0]), [X[:60, 0].mean(), X[60:, 0].mean()], atol=1e-6)
    assert sorted(len(v) for v in res[0]["groups"].values()) == [60, 60]
    groups = D.read_dict_vector(os.path.join(out, "centers_0"))
    assert len(groups) == 2
    assert len(open(os.path.join(out, "kmeans_0")).read().strip().split("\n")) == 2


def test_pagerank_matches_power_iteration(tmp_path):
    edges = [(1, 2), (1, 3), (2, 3), (3, 1), (4, 3), (4, 1), (5, 4)]
    p = tmp_path / "pr.txt"
    p.write_text("".join(f"{a},{b}\n" for a, b in edges) + "6,2147483648\n")
    res = LocalJob(2, 2).run(W.run_pagerank, (str(p), str(tmp_path / "pr"), 12), timeout_s=300)
    nodes = [1, 2, 3, 4, 5, 6]
    outdeg = {v: sum(1 for a, _ in edges if a == v) for v in nodes}
    outdeg[6] = 1
    pr = {v: 1.0 / 6 for v in nodes}
    for _ in range(12):
        pr = {v: 0.15 + 0.85 * sum(pr[a] / outdeg[a] for a, b in edges if b == v) for v in nodes}
    for v in nodes:
        assert abs(res[0][v] - pr[v]) < 1e-9
    dumped = D.read_dict_scalar(os.path.join(str(tmp_path / "pr"), "pagerank_0"))
    assert abs(dumped["3"] - pr[3]) < 1e-5


def test_max_vertex_value_and_pregel(tmp_path):
    p = tmp_path / "mvv.txt"
    p.write_text("1,2\n2,3\n3,1\n4,1\n7,4\n9,9\n")
    for use_pregel in (False, True):
        res = LocalJob(2, 1).run(W.run_mvv, (str(p), str(tmp_path / f"o{use_pregel}"), use_pregel),
                                 timeout_s=300)
        vals = {}
        for r in res:
            vals.update(r)
        assert vals == {"1": 7.0, "2": 7.0, "3": 7.0, "4": 7.0, "7": 7.0, "9": 9.0}


def _mf_data(tmp_path, nu=60, ni=40, nnz=1500, seed=1):
    rng = np.random.default_rng(seed)
    P, Q = rng.normal(0, 0.7, (nu, 3)), rng.normal(0, 0.7, (ni, 3))
    pairs = set()
    while len(pairs) < nnz:
        pairs.add((int(rng.integers(nu)), int(rng.integers(ni))))
    rows = [(u, i, float(np.clip(np.round(3 + P[u] @ Q[i]), 1, 5))) for u, i in sorted(pairs)]
    p = tmp_path / "ratings.txt"
    p.write_text("".join(f"{u} {i} 20140101 {r}\n" for u, i, r in rows))
    return str(p), rows


def test_mf_sgd_ssp_two_workers(tmp_path):
    inp, rows = _mf_data(tmp_path)
    out = str(tmp_path / "mf")
    res = LocalJob(2, 2).run(W.run_mf, (inp, out, 8, 12, True), timeout_s=300)
    curve = res[0]["curve"]
    assert curve[-1] < 0.95 * curve[0] and abs(res[0]["rmse"] - res[1]["rmse"]) < 1e-9
    assert abs(res[0]["miu"] - np.mean([r for _, _, r in rows])) < 1e-9
    Wd = D.read_dict_vector(os.path.join(out, "W_0"))
    Hd = D.read_dict_vector(os.path.join(out, "H_0"))
    assert len(Wd) == len({u for u, _, _ in rows}) and len(Hd) == len({i for _, i, _ in rows})
    assert len(next(iter(Wd.values()))) == 8
    miu = D.read_dict_scalar(os.path.join(out, "miu_0"))
    assert miu["rating_sz"] == len(rows)
    assert os.path.exists(os.path.join(out, "ubias_0")) and os.path.exists(os.path.join(out, "ibias_0"))


def test_als_matches_numpy_ridge(tmp_path):
    rng = np.random.default_rng(2)
    nu, ni, k = 30, 25, 4
    H = rng.normal(0, 1, (ni, k))
    (tmp_path / "H.txt").write_text("".join("%d\t%s\n" % (i, "|".join("%.8f" % v for v in H[i]))
                                            for i in range(ni)))
    rat = [(u, i, float(rng.normal())) for u in range(nu) for i in rng.choice(ni, 8, replace=False)]
    (tmp_path / "R.txt").write_text("".join(f"{u},{i},{r:.6f}\n" for u, i, r in rat))
    res = LocalJob(2, 1).run(W.run_als, (str(tmp_path / "R.txt"), str(tmp_path / "H.txt"),
                                         str(tmp_path / "als"), 0.3), timeout_s=300)
    Wall = {}
    for r in res:
        Wall.update(r["W"])
    assert len(Wall) == nu
    Hr = np.round(H, 8)
    for u in (0, 7, 29):
        its = [(i, r) for uu, i, r in rat if uu == u]
        Hs = Hr[[i for i, _ in its]]
        a = np.array([round(r, 6) for _, r in its])
        ref = np.linalg.solve(Hs.T @ Hs + 0.3 * np.eye(k), Hs.T @ a)
        assert np.allclose(Wall[u], ref, atol=1e-8)


def test_lda_two_workers_likelihood_improves(tmp_path):
    rng = np.random.default_rng(3)
    topics = [["apple", "pear", "plum", "fig"], ["cpu", "gpu", "ram", "disk"], ["sun", "moon", "star", "sky"]]
    docs = []
    for d in range(90):
        t = topics[d % 3]
        docs.append(" ".join(rng.choice(t, 30)))
    (tmp_path / "docs.txt").write_text("\n".join(docs) + "\n")
    out = str(tmp_path / "lda_")
    res = LocalJob(2, 2).run(W.run_lda, (str(tmp_path / "docs.txt"), out, 3, 25), timeout_s=300)
    assert res[0]["V"] == 12 and res[0]["tokens"] + res[1]["tokens"] == 2700
    assert res[0]["sum"] == 2700              # global topic sums count every token once
    ll = res[0]["loglik"]
    assert ll[-1] > ll[0] + 500
    lines = open(out + "0").read().strip().split("\n") + open(out + "1").read().strip().split("\n")
    assert len([l for l in lines if l]) == 3 and all("topic\t" in l and l.endswith("|") for l in lines if l)


def test_bsp_runs_are_deterministic(tmp_path):
    """Same input, same seed, BSP mode: two jobs write byte-identical model dumps."""
    rng = np.random.default_rng(2)
    X = np.concatenate([rng.normal(0, 0.3, (40, 3)), rng.normal(4, 0.3, (40, 3))])
    p = tmp_path / "km.txt"
    p.write_text("".join("%d\t%s\n" % (i, ",".join("%.6f" % v for v in X[i])) for i in range(80)))
    edges = [(1, 2), (1, 3), (2, 3), (3, 1), (4, 3), (4, 1), (5, 4), (2, 5)]
    g = tmp_path / "pr.txt"
    g.write_text("".join(f"{a},{b}\n" for a, b in edges))
    dumps = []
    for trial in range(2):
        out_k, out_p = str(tmp_path / f"km{trial}"), str(tmp_path / f"pr{trial}")
        LocalJob(2, 1).run(W.run_kmeans, (str(p), out_k, 2, 5), timeout_s=300)
        LocalJob(2, 2).run(W.run_pagerank, (str(g), out_p, 8), timeout_s=300)
        dumps.append((open(os.path.join(out_k, "centers_0"), "rb").read(),
                      open(os.path.join(out_k, "kmeans_0"), "rb").read(),
                      open(os.path.join(out_p, "pagerank_0"), "rb").read()))
    assert dumps[0] == dumps[1]
