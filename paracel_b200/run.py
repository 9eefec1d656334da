"""Worker-side driver: ``python -m paracel_b200.run <algorithm> --server_info S --cfg_file F``.

Every reference executable takes exactly ``--server_info`` and ``--cfg_file`` (e.g.
alg/classification/logistic_regression/lr_driver.cpp:26-32) and reads its parameters from the
JSON file; the keys accepted here are the ones of the reference drivers."""
from __future__ import annotations

import argparse
import os
import sys
from typing import Callable, Dict

from .parallel.comm import Comm, main_env
from .utils.misc import json_parser


def _lr(comm, info, pt):
    from .models.lr import logistic_regression
    s = logistic_regression(comm, info, pt.check_parse("training_input", str), pt.parse("output", str),
                            pt.get("update_file", ""), pt.get("update_func", ""), pt.get("method", "ipm"),
                            int(pt.get("rounds", 1)), float(pt.get("alpha", 0.002)), float(pt.get("beta", 0.1)),
                            bool(pt.get("debug", False)), int(pt.get("limit_s", 0)),
                            bool(pt.get("ssp_switch", False)))
    s.solve()
    print("final loss:", s.calc_loss())
    if pt.get("test_input"):
        print("test loss:", s.test(pt.get("test_input")))
    if pt.get("predict_input"):
        s.predict(pt.get("predict_input"))
    s.dump_result()
    return s


def _ridge(comm, info, pt):
    from .models.lr import ridge_regression
    s = ridge_regression(comm, info, pt.check_parse("training_input", str), pt.parse("output", str),
                         pt.get("update_file", ""), pt.get("update_func", ""), "ipm",
                         int(pt.get("rounds", 1)), float(pt.get("alpha", 0.002)), float(pt.get("beta", 0.1)))
    s.solve()
    print("final loss:", s.calc_loss())
    if pt.get("predict_input"):
        s.predict(pt.get("predict_input"))
    s.dump_result()
    return s


def _mf(comm, info, pt):
    from .models.mf import matrix_factorization
    s = matrix_factorization(comm, info, pt.check_parse("input", str), pt.get("predict_input", ""),
                             pt.parse("output", str), pt.get("update_file", ""),
                             pt.get("update_functions"), pt.get("filter_file", ""),
                             pt.get("filter_functions"), int(pt.get("k", 80)), int(pt.get("rounds", 1)),
                             float(pt.get("alpha", 0.005)), float(pt.get("beta", 0.01)),
                             bool(pt.get("debug", False)), bool(pt.get("ssp_switch", True)),
                             int(pt.get("limit_s", 3)))
    s.solve()
    print("rmse:", s.cal_rmse())
    s.predict()
    s.dump_result()
    return s


def _als(comm, info, pt):
    from .models.als import alternating_least_square_standard
    s = alternating_least_square_standard(comm, info, pt.check_parse("rating_input", str),
                                          pt.check_parse("factor_input", str), pt.parse("output", str),
                                          pt.get("pattern", "fmap"), float(pt.get("lambda", 0.1)))
    if pt.get("validate_input"):
        for lam, tr, va in s.validate(pt.get("validate_input"), pt.get("lambdas", [s.lam])):
            print(f"lambda {lam}: train rmse {tr} validate rmse {va}")
    else:
        s.solve()
        print("rmse:", s.cal_rmse())
    s.dump_result()
    return s


def _svd(comm, info, pt):
    from .models.svd import svd
    s = svd(comm, info, pt.check_parse("input", str), pt.parse("output", str), int(pt.parse("k")),
            pt.get("update_file", ""), pt.get("update_function", "svd_updater"))
    s.solve()
    s.dump_result()
    return s


def _lda(comm, info, pt):
    from .models.lda import LDAmodel
    s = LDAmodel(comm, info, pt.check_parse("input", str), pt.parse("output", str), float(pt.parse("alpha")),
                 float(pt.parse("beta")), int(pt.parse("k_topics")), int(pt.parse("iters")),
                 int(pt.get("top_words", 10)), pt.get("handle_file", ""), bool(pt.get("debug", False)))
    s.solve()
    s.save()
    return s


def _kmeans(comm, info, pt):
    from .models.kmeans import kmeans
    s = kmeans(comm, info, pt.check_parse("input", str), pt.parse("output", str), pt.get("type", "fvec"),
               int(pt.parse("kclusters")), pt.get("update_file", ""), pt.get("update_functions"),
               int(pt.get("rounds", 1)))
    s.solve()
    s.dump_result()
    return s


def _pagerank(comm, info, pt):
    from .models.pagerank import pagerank
    s = pagerank(comm, info, pt.check_parse("input", str), pt.parse("output", str), pt.get("handle_file", ""),
                 pt.get("update_function", "init_updater"), pt.get("filter_function", "pr_filter"),
                 int(pt.get("rounds", 1)), float(pt.get("damping_factor", 0.85)))
    s.solve()
    s.dump_result()
    return s


def _mvv(comm, info, pt):
    from .models.mvv import max_vertex_value
    s = max_vertex_value(comm, info, pt.check_parse("input", str), pt.parse("output", str),
                         pt.get("update_file", ""), pt.get("update_func", "max_updater"))
    s.solve()
    s.dump_result()
    return s


def _wc(comm, info, pt):
    from .models.wc import word_count
    s = word_count(comm, info, pt.check_parse("input", str), pt.get("output", ""), int(pt.get("topk", 10)),
                   pt.get("handle_file", ""), pt.get("update_function", "wc_updater"),
                   pt.get("filter_function", "wc_filter"))
    s.solve()
    s.print()
    return s


def _ssi(comm, info, pt):
    """Steady-state inversion, parallel over the left nodes (the reference has the serial tool only;
    same config keys as that tool: bigraph_input, distribution_input, output)."""
    from .models.ssi import steady_state_inversion
    s = steady_state_inversion(comm, info, pt.check_parse("bigraph_input", str), pt.get("output", ""),
                               pt.check_parse("distribution_input", str))
    s.solve()
    s.dump_result()
    return s


def _sim_dense(comm, info, pt):
    from .models.similarity import sim_dense
    a = pt.get("input") or pt.get("input_a")
    s = sim_dense(comm, info, a, pt.get("input_b") or a, pt.parse("output", str),
                  float(pt.get("simbar", 0.0)), int(pt.get("topk", 20)))
    s.solve()
    s.dump_result()
    return s


def _sim_sparse(comm, info, pt):
    from .models.similarity import sim_sparse_row
    s = sim_sparse_row(comm, info, pt.check_parse("input", str), pt.parse("output", str),
                       pt.get("format", "fsv"), int(pt.get("topk", 20)),
                       sim_bar=float(pt.get("sim_bar", 0.0)), sim_ubar=float(pt.get("sim_ubar", 1e30)))
    s.solve()
    s.dump_result()
    return s


def _adjust_ktop(comm, info, pt):
    from .models.adjust_ktop import adjust_ktop_s
    s = adjust_ktop_s(comm, info, pt.check_parse("rating_input", str), pt.get("fmt", "fsv"),
                      pt.check_parse("sim_input", str), int(pt.get("lower bound", 1)),
                      pt.parse("output", str))
    s.solve()
    print("rmse:", s.cal_rmse(), "original rmse:", s.cal_original_rmse())
    s.dump_result()
    return s


def _dtr(comm, info, pt):
    from .models.dtr import decision_tree_builder_factor
    s = decision_tree_builder_factor(comm, info, pt.check_parse("user_fac_input", str),
                                     pt.check_parse("item_fac_input", str), pt.parse("output", str),
                                     pt.get("handle_file", ""), int(pt.get("level", 3)),
                                     int(pt.get("tree_start_index", 0)), int(pt.get("tree_end_index", 0)))
    s.solve()
    s.dump()
    return s


def _l1(comm, info, pt, logistic=True):
    """Sparse L1 logistic regression / Lasso.  The reference ships these as serial tools only
    (tool/lr_l1_serial.cpp, tool/lasso_serial.cpp): without GPUs worker 0 runs the serial
    shooting solver; with ``--gpu`` the proximal-gradient device path takes over."""
    from .tool.lasso_serial import shooting_solver
    if comm.get_rank() == 0:
        s = shooting_solver(pt.check_parse("input", str), pt.parse("output", str), float(pt.get("lambda", 0.1)),
                            int(pt.get("rounds", 100)), logistic=logistic)
        s.solve()
        s.dump_result()
    comm.synchronize()
    return None


def _lasso(comm, info, pt):
    return _l1(comm, info, pt, logistic=False)


ALGORITHMS: Dict[str, Callable] = {
    "lr": _lr, "ridge": _ridge, "mf": _mf, "als": _als, "als_validate": _als, "svd": _svd, "gLDA": _lda,
    "lda": _lda, "kmeans": _kmeans, "pagerank": _pagerank, "mvv": _mvv, "wc": _wc,
    "sim_dense": _sim_dense, "ab_sim_dense": _sim_dense, "sim_sparse": _sim_sparse,
    "adjust_ktop_sparse": _adjust_ktop, "dtr": _dtr, "lr_l1": _l1, "lasso": _lasso,
    "steady_state_inversion": _ssi,
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="paracel_b200.run")
    ap.add_argument("algorithm", choices=sorted(ALGORITHMS))
    ap.add_argument("--server_info", required=True)
    ap.add_argument("--cfg_file", required=True)
    ap.add_argument("--resume", default="", help="checkpoint directory to continue from (device drivers)")
    ap.add_argument("--checkpoint", default="", help="directory to write a checkpoint to when the run ends")
    ap.add_argument("--metrics", action="store_true", help="write <output>/metrics.jsonl and a phase trace")
    a = ap.parse_args(argv)
    # the drivers see these through the environment, like the launcher's --gpu switch
    if a.resume:
        os.environ["PCL_RESUME"] = a.resume
    if a.checkpoint:
        os.environ["PCL_CHECKPOINT"] = a.checkpoint
    if a.metrics:
        os.environ["PCL_METRICS"] = "1"
    env = main_env()
    try:
        comm = Comm()
        driver = ALGORITHMS[a.algorithm]
        if os.environ.get("PCL_USE_GPU", "0") == "1":     # launcher started with --gpu
            import torch
            from .run_gpu import GPU_ALGORITHMS
            if torch.cuda.is_available() and a.algorithm in GPU_ALGORITHMS:
                driver = GPU_ALGORITHMS[a.algorithm]
        s = driver(comm, a.server_info, json_parser(a.cfg_file))
        comm.synchronize()
        closer = getattr(s, "close", None)
        if closer:
            closer()
    finally:
        env.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
