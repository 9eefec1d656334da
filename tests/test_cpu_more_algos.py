"""Remaining algorithms (similarity, adjust_ktop, decision tree, SVD) on 2 workers, and the
serial tools, against NumPy oracles."""
import json
import os

import numpy as np

from paracel_b200.launch.local import LocalJob
from workers import cpu_workers as W
from paracel_b200.utils import dump as D


def test_sim_dense_topk(tmp_path):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((40, 6))
    p = tmp_path / "items.csv"
    p.write_text("".join("%d,%s\n" % (i, ",".join("%.6f" % v for v in X[i])) for i in range(40)))
    res = LocalJob(2, 1).run(W.run_sim_dense, (str(p), str(tmp_path / "o"), 3), timeout_s=300)
    allr = {}
    for r in res:
        allr.update(r)
    Xn = np.round(X, 6)
    Xn = Xn / np.linalg.norm(Xn, axis=1, keepdims=True)
    S = Xn @ Xn.T
    np.fill_diagonal(S, -np.inf)
    for i in (0, 17, 39):
        top = np.argsort(-S[i])[:3]
        assert [j for j, _ in allr[i]] == top.tolist()
        assert abs(allr[i][0][1] - S[i, top[0]]) < 1e-9
    assert os.path.exists(str(tmp_path / "o" / "result_0"))


def test_sim_sparse_ring(tmp_path):
    rows = {1: {10: 1.0, 11: 2.0}, 2: {10: 2.0, 11: 4.0}, 3: {12: 1.0}, 4: {11: 1.0, 12: 1.0}}
    p = tmp_path / "g.csv"
    p.write_text("".join(f"{r},{c},{v}\n" for r, nb in rows.items() for c, v in nb.items()))
    res = LocalJob(2, 1).run(W.run_sim_sparse, (str(p), str(tmp_path / "o"), 2), timeout_s=300)
    allr = {}
    for r in res:
        allr.update(r)
    assert allr[1][0][0] == 2 and abs(allr[1][0][1] - 1.0) < 1e-9      # parallel rows
    assert allr[3][0][0] == 4
    sims = D.read_dict_vector if False else None
    assert os.path.exists(str(tmp_path / "o" / "similarities_0"))


def test_adjust_ktop(tmp_path):
    (tmp_path / "sim.txt").write_text("1\t2:0.9|3:0.5|4:0.1\n2\t1:0.9|3:0.4\n")
    (tmp_path / "rat.txt").write_text("1,100,4\n1,101,2\n2,100,4\n2,101,2\n3,100,1\n3,101,5\n4,100,3\n4,101,3\n")
    res = LocalJob(2, 1).run(W.run_adjust_ktop, (str(tmp_path / "rat.txt"), str(tmp_path / "sim.txt"),
                                                 str(tmp_path / "o")), timeout_s=300)
    kt = {}
    for r in res:
        kt.update(r["ktop"])
    # user 2 predicts user 1 perfectly (residual 0 is skipped as "no information"), adding
    # user 3 makes it worse, so a small neighbourhood wins
    assert set(kt) == {1, 2} and 1 <= kt[1] <= 3 and 1 <= kt[2] <= 2


def test_decision_tree_builder(tmp_path):
    rng = np.random.default_rng(1)
    U, I = rng.standard_normal((60, 4)), rng.standard_normal((25, 4))
    (tmp_path / "u.txt").write_text("".join("%d\t%s\n" % (i, "|".join("%.6f" % v for v in U[i])) for i in range(60)))
    (tmp_path / "i.txt").write_text("".join("%d\t%s\n" % (i, "|".join("%.6f" % v for v in I[i])) for i in range(25)))
    out = str(tmp_path / "o")
    res = LocalJob(2, 1).run(W.run_dtr, (str(tmp_path / "u.txt"), str(tmp_path / "i.txt"), out, 2),
                             timeout_s=300)
    assert res[0] == res[1] and len(res[0][0]) == 3 and len(res[0][1]) == 3
    assert res[0][0][0] != res[0][1][0]                    # tree k starts from the k-th best split
    lines = open(os.path.join(out, "tree_0")).read().strip().split("\n")
    assert lines[0].startswith("tree_0\t") and len(lines) == 2
    avg = open(os.path.join(out, "average_user_factor_0")).read().strip().split("\n")
    assert len(avg) == 3 and len(avg[0].split("|")) == 4


def test_svd_two_workers_matches_numpy(tmp_path):
    rng = np.random.default_rng(2)
    A = rng.standard_normal((30, 3)) @ np.diag([9.0, 4.0, 1.0]) @ rng.standard_normal((3, 12))
    (tmp_path / "a.csv").write_text("".join(f"{i},{j},{A[i, j]:.8f}\n" for i in range(30) for j in range(12)))
    res = LocalJob(2, 1).run(W.run_svd, (str(tmp_path / "a.csv"), str(tmp_path / "o"), 3), timeout_s=300)
    ref = np.linalg.svd(np.round(A, 8), compute_uv=False)[:3]
    assert np.allclose(res[0]["sigma"], ref, rtol=1e-6)
    sig = [float(x) for x in open(str(tmp_path / "o" / "SIGMA_0")).read().strip().split(",")]
    assert np.allclose(sig, ref, rtol=1e-5)
    # the serial tool (numpy only, no code shared with the parallel class) as oracle: same
    # singular values and, up to the sign of a column, the same left singular vectors per row id
    from paracel_b200.tool import svd_serial
    ser = svd_serial.solve(str(tmp_path / "a.csv"), str(tmp_path / "os"), 3, iters=15)
    assert np.allclose(ser.sigma, res[0]["sigma"], rtol=1e-6)
    from paracel_b200.utils.dump import files_merge, read_dict_vector
    files_merge(str(tmp_path / "o" / "U_*"), str(tmp_path / "U_par"))
    Up, Us = read_dict_vector(str(tmp_path / "U_par")), read_dict_vector(str(tmp_path / "os" / "U_0"))
    assert sorted(Up) == sorted(Us) and len(Up) == 30
    P = np.array([Up[r] for r in sorted(Up)], dtype=float)
    S = np.array([Us[r] for r in sorted(Up)], dtype=float)
    for c in range(3):
        assert min(np.abs(P[:, c] - S[:, c]).max(), np.abs(P[:, c] + S[:, c]).max()) < 1e-5


def test_steady_state_inversion_two_workers_matches_serial_tool(tmp_path):
    """The parallel class against the serial tool on a random bipartite graph whose target
    distribution is far from what the initial scores deliver."""
    from paracel_b200.tool.steady_state_inversion_serial import steady_state_inversion as serial
    from paracel_b200.utils.dump import files_merge
    rng = np.random.default_rng(5)
    nl, nr = 40, 12
    lines = []
    for i in range(nl):
        for j in rng.choice(nr, size=4, replace=False):
            lines.append(f"n{i}L,m{j}R,{rng.uniform(0.5, 3.0):.6f}\n")
    (tmp_path / "bg.csv").write_text("".join(lines))
    pl = rng.dirichlet(np.ones(nl))
    pr = rng.dirichlet(np.ones(nr) * 3.0)
    (tmp_path / "dis.csv").write_text("".join(f"n{i}L,{pl[i]:.10f}\n" for i in range(nl)) +
                                      "".join(f"m{j}R,{pr[j]:.10f}\n" for j in range(nr)))
    ser = serial(str(tmp_path / "bg.csv"), str(tmp_path / "dis.csv"), str(tmp_path / "os"))
    ser.solve()
    ser.dump_result()
    res = LocalJob(2, 1).run(W.run_ssi, (str(tmp_path / "bg.csv"), str(tmp_path / "dis.csv"), str(tmp_path / "op")),
                             timeout_s=300)
    assert res[0]["left"] + res[1]["left"] == nl and res[0]["left"] > 0 and res[1]["left"] > 0
    assert res[0]["score"] == res[1]["score"]
    for r, v in ser.score_new.items():
        assert abs(res[0]["score"][r] - v) <= 1e-8 * max(1.0, abs(v)), (r, v, res[0]["score"][r])
    # the scores moved, and the dumps agree line by line after merging the workers' parts
    assert any(abs(ser.score_new[f"m{j}R"] - pr[j]) > 1e-6 for j in range(nr))
    files_merge(str(tmp_path / "op" / "transfer_prob_matrix_*"), str(tmp_path / "tp_par"))
    par = sorted(open(str(tmp_path / "tp_par")).read().strip().split("\n"))
    one = sorted(open(str(tmp_path / "os" / "transfer_prob_matrix_0")).read().strip().split("\n"))
    assert len(par) == len(one) == nl
    for a, b in zip(par, one):
        ka, kb = a.split("\t")[0], b.split("\t")[0]
        assert ka == kb
        ea = dict(x.split(":") for x in a.split("\t")[1].split("|"))
        eb = dict(x.split(":") for x in b.split("\t")[1].split("|"))
        assert ea.keys() == eb.keys()
        assert all(abs(float(ea[k]) - float(eb[k])) < 1e-6 for k in ea)


def test_serial_tools(tmp_path):
    from paracel_b200.tool import datagen, gLDA_serial, kmeans_serial, lasso_serial, lr_serial, svd_serial
    from paracel_b200.tool.steady_state_inversion_serial import steady_state_inversion
    out = str(tmp_path / "out")
    # lr
    X, y, w = datagen.classification(str(tmp_path / "c.csv"), 800, 5)
    s = lr_serial.lr_serial(str(tmp_path / "c.csv"), out, rounds=300, alpha=0.5)
    s.solve()
    assert s.loss() < 0.5
    s.dump_result()
    assert len(open(os.path.join(out, "lr_theta_0")).read().split("|")) == 6
    # lasso recovers a sparse vector; L1-LR separates
    rng = np.random.default_rng(0)
    Xl = rng.standard_normal((300, 10))
    wt = np.zeros(10)
    wt[[1, 4]] = [2.0, -3.0]
    np.savetxt(str(tmp_path / "l.csv"), np.concatenate([Xl, (Xl @ wt)[:, None]], 1), delimiter=",", fmt="%.6f")
    for rigid in (False, True):
        ls = lasso_serial.shooting_solver(str(tmp_path / "l.csv"), out, lam=1.0, rounds=200, rigid=rigid)
        ls.solve()
        assert np.allclose(ls.rW, wt, atol=0.05)
        assert abs(ls.rW[0]) < 1e-3
    ls.dump_result()
    assert os.path.exists(os.path.join(out, "lasso_weight_0"))
    l1 = lasso_serial.shooting_solver(str(tmp_path / "c.csv"), out, lam=0.5, rounds=100, logistic=True)
    l1.solve()
    acc = np.mean((np.round(X, 6) @ l1.rW > 0) == (y > 0.5))
    assert acc > 0.7 and len(l1.check()) == 800
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps({"input": str(tmp_path / "c.csv"), "output": out, "lambda": 0.5, "rounds": 5}))
    lasso_serial.main_lr_l1(str(cfg))
    assert os.path.exists(os.path.join(out, "lr_l1_weight_0"))
    # kmeans
    Xk, lab = datagen.kmeans(str(tmp_path / "k.txt"), 200, 3, ncenters=2, seed=4)
    ks = kmeans_serial.kmeans_serial(str(tmp_path / "k.txt"), out, 2, 8)
    ks.solve()
    ks.dump_result()
    assert sum(len(v) for v in ks.groups.values()) == 200
    # lda
    datagen.lda(str(tmp_path / "d.txt"), 60, 40, 3, 30)
    g = gLDA_serial.gLDA_serial(str(tmp_path / "d.txt"), str(tmp_path / "lda_"), 0.5, 0.1, 3, 15)
    g.solve()
    g.save()
    assert g.loglik[-1] > g.loglik[0] and g.perplexity() > 1
    assert len(open(str(tmp_path / "lda_0")).read().strip().split("\n")) == 3
    # svd
    A = rng.standard_normal((15, 2)) @ rng.standard_normal((2, 8))
    (tmp_path / "a.csv").write_text("".join(f"{i},{j},{A[i, j]:.8f}\n" for i in range(15) for j in range(8)))
    sv = svd_serial.solve(str(tmp_path / "a.csv"), out, 2)
    assert np.allclose(sv.sigma, np.linalg.svd(np.round(A, 8), compute_uv=False)[:2], rtol=1e-6)
    U = D.read_dict_vector(os.path.join(out, "U_0"))
    assert len(U) == 15 and len(U["0"]) == 2
    # steady state inversion
    (tmp_path / "bg.csv").write_text("aL,xR,1.0\naL,yR,1.0\nbL,yR,2.0\n")
    (tmp_path / "dis.csv").write_text("aL,0.5\nbL,0.5\nxR,0.4\nyR,0.6\n")
    ss = steady_state_inversion(str(tmp_path / "bg.csv"), str(tmp_path / "dis.csv"), out)
    ss.solve()
    ss.dump_result()
    assert abs(ss.q("xR") - 0.4) < 2e-3 * 0.4 + 1e-4
    assert os.path.exists(os.path.join(out, "score_0")) and os.path.exists(os.path.join(out, "transfer_prob_matrix_0"))
    datagen.regression(str(tmp_path / "r.csv"), 50, 3)
    datagen.ratings(str(tmp_path / "rt.txt"), 20, 10, 100)
    datagen.graph(str(tmp_path / "g.txt"), 50, 200)
    datagen.main(["-m", "classification", "-o", str(tmp_path / "c2.csv"), "-n", "10", "-k", "2"])


def test_balltree_matches_brute_force(tmp_path):
    from paracel_b200.tool.balltree import (PyBalltree, PyQuery, balltree_search, balltree_search_with_dp,
                                            linear_search, linear_search_with_dp)
    rng = np.random.default_rng(5)
    items = rng.standard_normal((2000, 16))
    t = PyBalltree(items)
    t.build()
    assert t.node_count > 100
    for trial in range(20):
        q = PyQuery(rng.standard_normal(16), 5)
        got = balltree_search_with_dp(q, t)
        ref = np.argsort(-(items @ np.asarray(q.get_item())))[:5]
        assert [i for i, _ in got] == ref.tolist()
        assert balltree_search(q, t) == linear_search(q, t)
    assert t.last_visited < t.node_count                   # the bound prunes
    qb = PyQuery(items[3] * 10, 3, black_list=[3])
    assert 3 not in balltree_search(qb, t)
    qw = PyQuery(items[3], 2, white_list=[5, 9, 11])
    assert set(balltree_search(qw, t)) <= {5, 9, 11}
    assert linear_search_with_dp(qw, items)[0][0] in (5, 9, 11)
    t.pickle(str(tmp_path / "bt.txt"))
    t2 = PyBalltree(items)
    t2.build_from_file(str(tmp_path / "bt.txt"))
    q = PyQuery(rng.standard_normal(16), 4)
    assert balltree_search(q, t2) == balltree_search(q, t)
