#!/usr/bin/env python
"""Held-out RMSE per epoch of the MF-SGD kernel against the fp64 sequential pass, on Zipf ids
where the kernel's approximations (concurrency weights, per-CTA replicas of the hottest item
rows) are active.  One JSON line per configuration.

    python benchmarks/bench_mf_parity.py                         # default kernel settings + oracles
    python benchmarks/bench_mf_parity.py --hot-mix 1 0.5 0.25 0.125 0.0625 --hot-rows 106 0

Oracles: `seq_shuffled` visits the training ratings in random order, `seq_by_user` user by user
(users in random order), which is how the reference walks its bigraph
(alg/recommendation/matrix_factorization/mf.hpp:313).  All runs start from the same factors.
"""
import argparse
import json
import math
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--users", type=int, default=50_000)
    ap.add_argument("--items", type=int, default=10_000)
    ap.add_argument("--nnz", type=int, default=5_000_000)
    ap.add_argument("--rank", type=int, default=128)
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--zipf-s", type=float, default=1.1)
    ap.add_argument("--hot-mix", type=float, nargs="*", default=[-1.0], help="negative: the model's default")
    ap.add_argument("--hot-rows", type=int, nargs="*", default=[106])
    ap.add_argument("--no-oracle", action="store_true")
    args = ap.parse_args()
    from paracel_b200._core import core
    from paracel_b200.models.mf_gpu import MfSgdGpu
    from paracel_b200.utils.synth import MfRatingStream
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    nu, ni, nnz, k = args.users, args.items, args.nnz, args.rank
    u, i, r = MfRatingStream(nu, ni, nnz, s=args.zipf_s, seed=1, device=dev, chunk=nnz).chunk_at(0)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    perm = torch.randperm(nnz, device=dev, generator=g)
    nh = nnz // 20
    hu, hi, hr = u[perm[:nh]], i[perm[:nh]], r[perm[:nh]]
    tu, ti, tr = u[perm[nh:]], i[perm[nh:]], r[perm[nh:]]
    marks = [e for e in (1, 2, 5, 10, 20, 50) if e <= args.epochs]
    init = None
    for mix in args.hot_mix:
        for hot in args.hot_rows:
            m = MfSgdGpu(nu, ni, k=k, alpha=0.005, beta=0.02, rounds=args.epochs, staleness=0, ssp=False,
                         device=dev, seed=3, hot_rows=hot, hot_mix=(mix if mix >= 0 else None))
            m.load_ratings(tu, ti, tr)
            m.init_parameters()
            if init is None:
                init = (m.Wt.shard[:nu, :k].double().cpu().numpy().copy(), m.Ht.shard[:ni, :k].double().cpu().numpy().copy(),
                        m.but.shard[:nu].double().cpu().numpy().copy(), m.bit.shard[:ni].double().cpu().numpy().copy(), m.mu)
            out = {"impl": "gpu", "hot_mix": m.hot_mix, "hot_rows": m.hot_T, "min_user_weight": float(m.su.min()),
                   "min_item_weight": float(m.si.min()), "heldout_rmse": {}}
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            for e in range(1, args.epochs + 1):
                if e == 2:
                    ev[0].record()
                m.round()
                if e == 2:
                    ev[1].record()
                    torch.cuda.synchronize()
                    out["ms_per_epoch"] = ev[0].elapsed_time(ev[1])
                if e in marks:
                    sse, cnt = m.heldout_sse(hu, hi, hr)
                    out["heldout_rmse"][e] = math.sqrt(sse / cnt)
            m.paracel_check()
            m.free()
            print(json.dumps(out), flush=True)
    if args.no_oracle or init is None:
        return
    W0, H0, bu0, bi0, mu = init
    hu_c, hi_c, hr_c = hu.cpu().numpy(), hi.cpu().numpy(), hr.double().cpu().numpy()
    tu_c, ti_c, tr_c = tu.cpu().numpy().astype(np.int64), ti.cpu().numpy().astype(np.int64), tr.double().cpu().numpy()
    orders = {"seq_shuffled": np.arange(tu_c.size),
              "seq_by_user": np.argsort(np.random.default_rng(0).permutation(nu)[tu_c], kind="stable")}
    for name, order in orders.items():
        uu, ii, rr = (np.ascontiguousarray(x[order]) for x in (tu_c, ti_c, tr_c))
        W, H, bu, bi = W0.copy(), H0.copy(), bu0.copy(), bi0.copy()
        out = {"impl": name, "heldout_rmse": {}}
        t0 = time.time()
        for e in range(1, args.epochs + 1):
            core().mf_sgd_pass(uu, ii, rr, W, H, bu, bi, mu, 0.005, 0.02)
            if e in marks:
                p = np.clip(mu + bu[hu_c] + bi[hi_c] + (W[hu_c] * H[hi_c]).sum(1), 1, 5)
                out["heldout_rmse"][e] = float(np.sqrt(((p - hr_c) ** 2).mean()))
        out["s_per_epoch_cpu"] = (time.time() - t0) / args.epochs
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
