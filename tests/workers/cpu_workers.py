"""Worker bodies of the multi-process CPU tests (gloo ranks + host parameter servers)."""
from __future__ import annotations

import os
import time


def comm_primitives(comm, server_info):
    """Every Comm primitive with assertions (the reference's test_comm.cpp only prints)."""
    import numpy as np
    rk, sz = comm.get_rank(), comm.get_size()
    out = {}
    # send / recv of builtin, containers, triples with empty elements, dicts
    if rk == 0:
        comm.send(7, 1)
        comm.send([1.5, 2.5], 1)
        comm.send("hello", 1)
        comm.send([("a", "b", 1.0), ("c", "d", 2.0)], 1)
        comm.send([[], [("x", "y", 3.0)]], 1)
        comm.send({"k": [1, 2]}, 1)
    elif rk == 1:
        out["p2p"] = [comm.recv(0) for _ in range(6)]
    comm.synchronize()
    # isend + sendrecv ring
    right, left = (rk + 1) % sz, (rk + sz - 1) % sz
    out["ring"] = comm.sendrecv({"from": rk}, right, left)
    # bcast
    out["bcast"] = comm.bcast([rk, "x"] if rk == 0 else None, 0)
    # bcastring: union of everybody's list
    seen = []
    comm.bcastring([rk, rk * 10], lambda v: seen.extend(v))
    out["bcastring"] = sorted(seen)
    # alltoall with variable sizes
    got = comm.alltoall([[rk] * (d + 1) for d in range(sz)])
    out["alltoall"] = got
    acc = []
    comm.alltoallring([[rk, d] for d in range(sz)], lambda v: acc.append(v))
    out["alltoallring"] = sorted(acc)
    # allreduce on every supported kind
    out["ar_int"] = comm.allreduce(rk + 1)
    out["ar_float"] = comm.allreduce(0.5)
    out["ar_list"] = comm.allreduce([1.0, float(rk)])
    out["ar_np"] = comm.allreduce(np.ones(3) * rk).tolist()
    # treereduce with scalar and dict combiners
    out["tree_sum"] = comm.treereduce(rk + 1, lambda a, b: a + b, 0)

    def merge(a, b):
        c = dict(a)
        for k, v in b.items():
            c[k] = c.get(k, 0) + v
        return c
    out["tree_dict"] = comm.treereduce({"n": 1, str(rk): 1}, merge, 0)
    # split into even / odd ranks
    sub = comm.split(rk % 2)
    out["split"] = (sub.get_rank(), sub.get_size(), sub.allreduce(1))
    comm.synchronize()
    return out


def ps_ops(comm, server_info):
    """The whole operation table through paralg."""
    from paracel_b200.paralg import paralg
    from paracel_b200.ps.handlers import register_handler
    pt = paralg(server_info, comm)
    rk, sz = comm.get_rank(), comm.get_size()
    out = {}
    pt.paracel_write(f"k{rk}", [1.0, 2.0])
    pt.paracel_write_multi({f"m{rk}_{i}": i for i in range(5)})
    pt.paracel_sync()
    out["read"] = pt.paracel_read(f"k{(rk + 1) % sz}")
    out["contains"] = (pt.paracel_contains("k0"), pt.paracel_contains("nope"))
    out["multi"] = pt.paracel_read_multi([f"m0_{i}" for i in range(5)])
    out["multi_dict"] = pt.paracel_read_multi(["m0_1", "missing"], as_dict=True)
    try:
        pt.paracel_read("missing")
        out["missing"] = "no error"
    except KeyError:
        out["missing"] = "KeyError"
    # bupdate with a built-in handler name of the reference and with a python handler file
    pt.paracel_bupdate("theta", [1.0, 1.0, 1.0], "", "lr_theta_update")
    pt.paracel_sync()
    out["theta"] = pt.paracel_read("theta")
    hfile = os.path.join(os.path.dirname(__file__), "sample_handlers.py")
    pt.paracel_bupdate("prod", 2, hfile, "multiply")
    pt.paracel_sync()
    out["prod"] = pt.paracel_read("prod")
    fut = pt.paracel_update("cnt", 1, "", "cnt_updater")
    out["update_future"] = fut.result()
    pt.paracel_sync()
    out["cnt"] = pt.paracel_read("cnt")
    pt.paracel_bupdate_multi({f"bm{i}": 1 for i in range(3)}, "", "add")
    pt.paracel_bupdate_multi([f"bm{i}" for i in range(3)], [1, 1, 1], "", "add")
    pt.paracel_sync()
    out["bm"] = pt.paracel_read_multi([f"bm{i}" for i in range(3)])
    out["special"] = sorted(pt.paracel_read_special("", "prefix:bm").keys())
    out["special_py"] = sorted(pt.paracel_read_special(hfile, "starts_with_k").keys())
    out["topk"] = pt.paracel_read_topk_with_key_filter(2, "", "prefix:m0_")
    pt.paracel_sync()
    if rk == 0:
        pt.paracel_remove("k0")
        pt.paracel_remove_special("", "prefix:m1_")
    pt.paracel_sync()
    out["after_remove"] = (pt.paracel_contains("k0"), pt.paracel_contains("m1_2"), pt.paracel_contains("m0_2"))
    out["all_keys"] = len(pt.paracel_readall())
    pt.paracel_sync()
    pt.close()
    return out


def ssp_bound(comm, server_info, limit_s, iters, slow_rank, delay):
    """A fast worker is never more than limit_s clocks ahead of the slowest running one;
    finished workers stop being waited for."""
    from paracel_b200.paralg import paralg
    pt = paralg(server_info, comm, rounds=iters, limit_s=limit_s, ssp_switch=True)
    rk = comm.get_rank()
    pt.paracel_write("w", 0.0)
    pt.paracel_sync()
    ahead = []
    for it in range(iters):
        pt.paracel_read("w")
        sc = pt.ps_obj.kvm[0].pull_int("server_clock")
        ahead.append(pt.clock - sc)
        if rk == slow_rank:
            time.sleep(delay)
        pt.paracel_bupdate("w", 1.0, "", "add")
        pt.iter_commit()
    final = pt.paracel_read("w")   # clock == total_iters: always pulls
    pt.paracel_sync()
    total = pt.paracel_read("w")
    pt.close()
    return {"max_ahead": max(ahead), "final": final, "total": total, "clock": pt.clock}


def ssp_withheld_commit(comm, server_info):
    """Fault injection on the host: rank 1 never commits.  Rank 0's staleness wait must end
    with ParacelTimeout, not hang."""
    from paracel_b200.paralg import ParacelTimeout, paralg
    pt = paralg(server_info, comm, rounds=10, limit_s=1, ssp_switch=True, wait_timeout_s=0.5)
    rk = comm.get_rank()
    pt.paracel_write(f"x{rk}", 1.0)
    pt.paracel_sync()
    res = "no timeout"
    if rk == 0:
        try:
            for it in range(5):
                pt.paracel_read("x0")
                pt.iter_commit()
        except ParacelTimeout as e:
            res = "timeout at clock %d" % pt.clock
    pt.paracel_sync()
    pt.close()
    return res


def run_lr(comm, server_info, inp, out, method, ssp, rounds=10):
    from paracel_b200.models.lr import logistic_regression
    m = logistic_regression(comm, server_info, inp, out, method=method, rounds=rounds, alpha=0.01,
                            beta=0.0, seed=comm.get_rank(), limit_s=1 if ssp else 0, ssp_switch=ssp)
    t = time.time()
    m.solve()
    dt = time.time() - t
    loss = m.calc_loss()
    m.predict(inp)
    m.dump_result()
    m.close()
    return {"loss": loss, "seconds": dt, "seconds_learn": m.seconds_learn, "seconds_load": m.seconds_load,
            "n": int(m.samples.shape[0]), "theta": m.theta.tolist()}


def run_wc(comm, server_info, inp, topk, variant="learning"):
    from paracel_b200.models.wc import word_count
    m = word_count(comm, server_info, inp, "", topk)
    lines = m.paracel_load(inp)
    m.paracel_sync()
    getattr(m, variant)(lines)
    m.paracel_sync()
    m.close()
    return m.result


def run_kmeans(comm, server_info, inp, out, k, rounds):
    from paracel_b200.models.kmeans import kmeans
    m = kmeans(comm, server_info, inp, out, kclusters=k, rounds=rounds)
    m.solve()
    m.dump_result()
    m.close()
    return {"clusters": m.clusters, "groups": m.groups}


def run_pagerank(comm, server_info, inp, out, rounds):
    from paracel_b200.models.pagerank import pagerank
    m = pagerank(comm, server_info, inp, out, rounds=rounds)
    m.solve()
    m.dump_result()
    m.close()
    return m.kvmap


def run_mvv(comm, server_info, inp, out, use_pregel=False):
    if use_pregel:
        from paracel_b200.pregel import max_vertex_value_pregel
        from paracel_b200.utils.ext import str_split
        m = max_vertex_value_pregel(comm, server_info, inp, out, lambda l: str_split(l, ","))
        m.run_supersteps()
        m.dump_result("vertex_val_")
        m.pt.close()
        return m.vertex_val_map
    from paracel_b200.models.mvv import max_vertex_value
    m = max_vertex_value(comm, server_info, inp, out)
    m.solve()
    m.dump_result()
    m.close()
    return m.vertex_val_map


def run_mf(comm, server_info, inp, out, k, rounds, ssp):
    from paracel_b200.models.mf import matrix_factorization
    m = matrix_factorization(comm, server_info, inp, "", out, k=k, rounds=rounds, alpha=0.01, beta=0.02,
                             debug=True, ssp_switch=ssp, limit_s=2)
    m.solve()
    r = m.cal_rmse()
    m.dump_result()
    m.close()
    return {"rmse": r, "curve": m.loss_error_train, "miu": m.miu}


def run_als(comm, server_info, rating, factor, out, lam):
    from paracel_b200.models.als import alternating_least_square_standard
    m = alternating_least_square_standard(comm, server_info, rating, factor, out, "fmap", lam)
    m.solve()
    r = m.cal_rmse()
    m.dump_result()
    m.close()
    return {"rmse": r, "W": m.W}


def run_lda(comm, server_info, inp, out, k, iters):
    from paracel_b200.models.lda import LDAmodel
    m = LDAmodel(comm, server_info, inp, out, alpha=0.5, beta=0.1, k_topics=k, iters=iters, top_words=5,
                 debug=True, seed=3)
    m.solve()
    m.save()
    m.close()
    return {"loglik": m.loglik, "V": m.V, "tokens": int(m.T), "sum": int(m.topic_sum.sum())}


def run_sim_dense(comm, server_info, inp, out, ktop):
    from paracel_b200.models.similarity import sim_dense
    m = sim_dense(comm, server_info, inp, inp, out, simbar=0.0, ktop=ktop)
    m.solve()
    m.dump_result()
    m.close()
    return m.result


def run_sim_sparse(comm, server_info, inp, out, topk):
    from paracel_b200.models.similarity import sim_sparse_row
    m = sim_sparse_row(comm, server_info, inp, out, "fsv", topk, sim_bar=0.0)
    m.solve()
    m.dump_result()
    m.close()
    return {k: [(j, s) for s, j in sorted(h, reverse=True)] for k, h in m.sim_result.items()}


def run_adjust_ktop(comm, server_info, rating, sim, out):
    from paracel_b200.models.adjust_ktop import adjust_ktop_s
    m = adjust_ktop_s(comm, server_info, rating, "fsv", sim, 1, out)
    m.solve()
    r = m.cal_rmse()
    m.dump_result()
    m.close()
    return {"ktop": m.ktop_result, "rmse": r}


def run_dtr(comm, server_info, ufac, ifac, out, level):
    from paracel_b200.models.dtr import decision_tree_builder_factor
    m = decision_tree_builder_factor(comm, server_info, ufac, ifac, out, "", level, 0, 1)
    m.solve()
    m.dump()
    m.close()
    return m.trees


def run_svd(comm, server_info, inp, out, k):
    from paracel_b200.models.svd import svd
    m = svd(comm, server_info, inp, out, k=k, iters=15)
    m.solve()
    m.dump_result()
    m.close()
    return {"sigma": m.sigma.tolist()}


def run_ssi(comm, server_info, graph, dis, out):
    from paracel_b200.models.ssi import steady_state_inversion
    m = steady_state_inversion(comm, server_info, graph, out, dis)
    m.solve()
    m.dump_result()
    res = {"score": dict(zip(m.right, m.score.tolist())), "sweeps": m.sweeps, "left": len(m.left)}
    m.close()
    return res


def checkpoint_resume(comm, server_info, inp, ckpt, phase):
    """LR (dgd, deterministic) for 6 rounds at once, or 3 rounds + checkpoint, or resume + 3."""
    import numpy as np
    from paracel_b200.models.lr import logistic_regression
    from paracel_b200.utils import checkpoint as C

    class resumable(logistic_regression):
        def _init_theta(self, dim):
            if phase == "resume":
                self.paracel_register_bupdate(self.update_file, self.update_func)
                return
            self.theta = np.full(dim, 0.5)
            self.paracel_write("theta", self.theta.tolist())
            self.paracel_register_bupdate(self.update_file, self.update_func)

    rounds = 6 if phase == "full" else 3
    m = resumable(comm, server_info, inp, "", method="dgd", rounds=rounds, alpha=1e-4, beta=0.0, seed=1)
    if phase == "resume":
        C.load_servers(m, ckpt)
        meta = C.load_meta(ckpt)
        assert meta["rounds_done"] == 3 and meta["world"] == comm.get_size()
    m.solve()
    if phase == "first":
        C.save_servers(m, ckpt)
        if comm.get_rank() == 0:
            C.save_meta(ckpt, {"rounds_done": 3, "world": comm.get_size()})
        C.save_rank_state(ckpt, comm.get_rank(), {"theta": m.theta, "rank": comm.get_rank()})
    theta = m.theta.tolist()
    m.close()
    return theta
