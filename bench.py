#!/usr/bin/env python
"""Headline benchmark: rating updates/s of matrix-factorisation SGD.

Config (synthetic, seeded): 1,000,000 users x 200,000 items, 200 M (user, item)
pairs drawn Zipf(1.1), ratings round(clip(p.q + N(0, 0.5), 1, 5)) from rank-16
latents; model rank 128 fp32, lr 0.005, L2 0.02, SSP staleness 2.  The total
work is fixed, so the scaling over GPUs is strong scaling.

One step = one training round of the public API: `MfSgdGpu` is a `paralg`
subclass and `round()` is `paracel_read_multi` (SSP wait + pull of the local
rows from the HBM shards), one SGD pass over all local ratings,
`paracel_bupdate_multi` (push of the weighted deltas to the owners) and
`iter_commit`.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3

Rank 0 prints one JSON line.  `value` is device-timed (CUDA events, max over
ranks) with the ratings resident in HBM; `e2e` repeats the measurement with the
ratings streamed from pinned host memory every round and the round's running
RMSE read back to the host.  `step_ms` gives the spread of the single steps
(an event after every step) and `heldout_rmse` the error on 2 M pairs drawn
from the same distribution that no rank trains on, after all epochs run.

`--impl reference` drives an installed build of the reference (looked up under
baseline/_ref) through its own executables; when none is installed it prints
one line saying what is missing.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time



def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_torch"])
    ap.add_argument("--users", type=int, default=1_000_000)
    ap.add_argument("--items", type=int, default=200_000)
    ap.add_argument("--nnz", type=int, default=200_000_000)
    ap.add_argument("--rank", type=int, default=128)
    ap.add_argument("--alpha", type=float, default=0.005)
    ap.add_argument("--beta", type=float, default=0.02)
    ap.add_argument("--staleness", type=int, default=2)
    ap.add_argument("--seed", type=int, default=20240611)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--spread-above", type=float, default=0.25,
                    help="ids holding more than this fraction of one group's share are dealt over all "
                         "ranks of the grid row / column (0: never)")
    ap.add_argument("--phases", action="store_true",
                    help="after the timed steps run two extra rounds with per-phase device timing")
    ap.add_argument("--no-balance", action="store_true")
    ap.add_argument("--hot-mix", type=float, default=-1.0, help="concurrency damping (negative: the model's default)")
    ap.add_argument("--sgd-blocks", type=int, default=0)
    ap.add_argument("--hot-rows", type=int, default=106)
    ap.add_argument("--variant", type=int, default=0, help="SGD kernel: 0 automatic (16 lanes per rating at rank 128), 1: 32 lanes per rating, "
                         "2: experimental 8 lanes per rating, 3: 16 lanes per rating")
    ap.add_argument("--chunks-per-flush", type=int, default=8)
    ap.add_argument("--zipf-s", type=float, default=1.1)
    ap.add_argument("--heldout", type=int, default=2_000_000,
                    help="pairs drawn like the training pairs but never trained on (0: skip)")
    ap.add_argument("--grid", default="", help="rank grid ROWSxCOLS of the rating partition (default: the "
                    "factorisation with the fewest factor rows per rank)")
    ap.add_argument("--overlap-push", type=int, default=-1,
                    help="1: push + commit on a side stream under the next SGD pass; 0: in line; "
                         "-1: the model's default")
    return ap.parse_args()


def main():
    args = parse_args()
    if args.impl == "reference":
        # launched like the other arm (one process per GPU under torchrun): the first rank alone
        # drives the reference's own launcher and prints the line
        if int(os.environ.get("RANK", "0")) == 0:
            from benchmarks.reference_arm import run_reference_arm
            print(json.dumps(run_reference_arm(args)))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun",
                  file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print("bench.py needs a CUDA device", file=sys.stderr)
        return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                device_id=dev)

    from paracel_b200.ops import _lib
    from paracel_b200.utils.clocks import ClockSampler
    from paracel_b200.utils.synth import MfRatingStream

    if args.impl == "nccl_torch":
        from paracel_b200.baselines.mf_nccl_torch import MfSgdNcclTorch as Model
    else:
        from paracel_b200.models.mf_gpu import MfSgdGpu as Model
    from paracel_b200.models.mf_gpu import balanced_groups, grid_rank

    K, Wm = args.steps, args.warmup
    total_rounds = 2 * (K + Wm) + 4
    t_setup = time.time()
    model = Model(args.users, args.items, k=args.rank, alpha=args.alpha, beta=args.beta,
                  rounds=total_rounds, staleness=args.staleness, ssp=True, seed=args.seed,
                  hot_mix=(args.hot_mix if args.hot_mix >= 0 else None), sgd_blocks=args.sgd_blocks, device=dev,
                  hot_rows=args.hot_rows, chunks_per_flush=args.chunks_per_flush,
                  variant=args.variant,
                  **({"grid": tuple(int(x) for x in args.grid.split("x"))} if args.grid and args.impl == "ours" else {}))
    if args.overlap_push >= 0 and hasattr(model, "overlap_push"):
        model.overlap_push = bool(args.overlap_push)

    # ---- data: every rank regenerates the same global stream and keeps its block
    stream = MfRatingStream(args.users, args.items, args.nnz, s=args.zipf_s, seed=args.seed,
                            device=dev)
    if world > 1 and not args.no_balance:
        cu, ci = stream.counts()
        ugrp = balanced_groups(cu, model.npx, spread_above=args.spread_above)
        igrp = balanced_groups(ci, model.npy, spread_above=args.spread_above)
    else:
        ar_u = torch.arange(args.users, device=dev)
        ar_i = torch.arange(args.items, device=dev)
        ugrp = (ar_u % model.npx).to(torch.int32)
        igrp = (ar_i % model.npy).to(torch.int32)
    us, is_, rs = [], [], []
    for u, i, r in stream:
        if world > 1:
            keep = grid_rank(u, i, ugrp, igrp, model.npx, model.npy) == rank
            u, i, r = u[keep], i[keep], r[keep]
        us.append(u.to(torch.int32))
        is_.append(i.to(torch.int32))
        rs.append(r.to(torch.float16))
    u = torch.cat(us).to(torch.int64)
    i = torch.cat(is_).to(torch.int64)
    r = torch.cat(rs).to(torch.float32)
    # held-out pairs: one more chunk of the same stream, split evenly over the ranks
    held = None
    if args.heldout > 0:
        hg = torch.Generator(device=dev)
        hg.manual_seed(args.seed * 1000003 + 999_983)
        from paracel_b200.utils.synth import zipf_draw
        hu = zipf_draw(stream.cdf_u, args.heldout, hg)
        hi = zipf_draw(stream.cdf_i, args.heldout, hg)
        hr = (stream.P[hu] * stream.Q[hi]).sum(1) + stream.noise * torch.randn(args.heldout, device=dev, generator=hg)
        hr = torch.round(hr.clamp_(1.0, 5.0))
        lo_h, hi_h = rank * args.heldout // world, (rank + 1) * args.heldout // world
        held = (hu[lo_h:hi_h].clone(), hi[lo_h:hi_h].clone(), hr[lo_h:hi_h].clone())
        del hu, hi, hr
    del us, is_, rs, stream
    local_nnz = u.numel()
    model.load_ratings(u, i, r)
    del u, i, r
    torch.cuda.empty_cache()
    model.init_parameters()
    t_setup = time.time() - t_setup

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def heldout_rmse():
        if held is None or not hasattr(model, "heldout_sse"):
            return None
        barrier()
        sse, cnt = model.heldout_sse(*held)
        t = torch.tensor([sse, cnt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t)
        barrier()
        return float((t[0] / t[1].clamp(min=1.0)).sqrt().item())

    def timed(n_steps, read_result):
        """Total device time of n_steps rounds (max over ranks) and the time of every single
        step (an event after each one; per step the max over ranks)."""
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)]
        l0 = _lib.launches()
        ev[0].record()
        last = None
        pending = None
        for j in range(n_steps):
            res = model.round()
            ev[j + 1].record()
            if read_result:
                # device -> host read of every step's result: the 8-byte copy into pinned memory is
                # queued behind the step's SGD pass; the host consumes it while the next step,
                # already queued, runs
                if not hasattr(res, "sse"):          # a model without result handles: read in place
                    last = float(model.sse.item())
                    continue
                if pending is not None:
                    last = pending.sse()
                pending = res
        if pending is not None:
            last = pending.sse()
        torch.cuda.synchronize()
        ms = torch.tensor([ev[0].elapsed_time(ev[-1])] +
                          [ev[j].elapsed_time(ev[j + 1]) for j in range(n_steps)],
                          dtype=torch.float64, device=dev)
        barrier()
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        steps = sorted(ms[1:].tolist())
        spread = {"median": steps[len(steps) // 2], "min": steps[0], "max": steps[-1],
                  "mean": sum(steps) / len(steps)}
        return float(ms[0].item()), _lib.launches() - l0, last, spread

    # ---- device-timed: ratings resident in HBM
    # clocks are sampled every 50 ms from the first warm-up step to the end of the timed steps
    # (a timed region of a few steps can be shorter than one sampling period)
    rmse0 = heldout_rmse()
    sampler = ClockSampler(local_rank, period_ms=50).start() if rank == 0 else None
    for _ in range(Wm):
        model.round()
    ms, launches, _, step_ms = timed(K, False)
    clocks = sampler.stop() if sampler else None
    model.paracel_check()
    run_rmse = model.running_rmse()
    if clocks and clocks.get("sm_mhz"):
        step_ms["median_ms_x_sm_mhz"] = step_ms["median"] * clocks["sm_mhz"]
    value = args.nnz * K / (ms * 1e-3)
    phases = None
    if args.phases and hasattr(model, "phase_times_ms"):   # extra untimed rounds, diagnostics only
        barrier()
        model.phase_timing = True
        for _ in range(2):
            model.round()
        phases = model.phase_times_ms()
        model.phase_timing = False
        if world > 1:
            allp = [None] * world
            dist.all_gather_object(allp, phases)
            phases = {"rank0": phases,
                      "sgd_ms_per_rank": [round(p.get("sgd", 0.0), 3) for p in allp]}
        barrier()

    # ---- end to end: ratings streamed from pinned host memory each round
    e2e = None
    if not args.no_e2e and hasattr(model, "offload_ratings"):
        model.offload_ratings()
        for _ in range(Wm):
            res = model.round()
            res.sse() if hasattr(res, "sse") else float(model.sse.item())
        ms2, _, last, step_ms2 = timed(K, True)
        model.paracel_check()
        e2e = {"value": args.nnz * K / (ms2 * 1e-3), "unit": "rating updates/s",
               "ms_per_step": ms2 / K, "step_ms": step_ms2,
               "h2d_bytes_per_step": int(model.h2d_bytes), "d2h_bytes_per_step": 8,
               "result_read": "every step's loss is copied to pinned host memory behind its SGD pass "
                              "and read by the host while the next step, already queued, runs"}
    final_rmse = model.running_rmse()
    epochs_run = (2 * (K + Wm) if e2e is not None else (K + Wm)) + (2 if phases is not None else 0)
    rmse1 = heldout_rmse()

    factor_mb = ((model.lu.numel() + model.li.numel()) * getattr(model, "D", args.rank) * 4 / 1e6
                 if hasattr(model, "lu") and hasattr(model, "li") else (args.users + args.items) * args.rank * 4 / 1e6 / world)
    mx = torch.tensor([local_nnz], dtype=torch.int64, device=dev)
    mn = mx.clone()
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    if rank == 0:
        out = {
            "metric": "rating updates/s (MF-SGD)",
            "value": value,
            "unit": "rating updates/s",
            "n_gpus": world,
            "steps": K,
            "warmup": Wm,
            "ms_per_step": ms / K,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp32",
            "data": "synthetic (seeded Zipf(1.1) pairs, rank-16 latent ratings), random-init factors",
            "impl": args.impl,
            "config": {
                "model": "biased MF, SGD, rank %d fp32" % args.rank,
                "users": args.users, "items": args.items, "ratings": args.nnz,
                "global_batch": args.nnz, "seq_len": None,
                "lr": args.alpha, "l2": args.beta, "ssp_staleness": args.staleness,
                "parallelism": "ps-shards-in-hbm x fsmap %dx%d" % (model.npx, model.npy),
                "l2_policy": "inputs larger than L2 (126 MB): per rank %.0f MB of ratings are streamed and "
                             "%.0f MB of factor rows are read and updated every step"
                             % (local_nnz * (getattr(model, "packed_bits", 32) / 8 + 0.375) / 1e6, factor_mb),
                "ratings_per_rank_max": int(mx.item()), "ratings_per_rank_min": int(mn.item()),
            },
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches,
            "step_ms": step_ms,
            "heldout_rmse": rmse1, "heldout_rmse_initial": rmse0, "heldout_pairs": args.heldout,
            "epochs_before_heldout_rmse": epochs_run,
            "phases_ms": phases,
            "running_rmse_device_phase": run_rmse,
            "running_rmse_final": final_rmse,
            "setup_s": t_setup,
        }
        print(json.dumps(out))
    model.free()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
