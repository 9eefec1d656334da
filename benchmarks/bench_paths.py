#!/usr/bin/env python
"""Micro-benchmarks of the fused parameter-server paths, one kernel family at a time.

    python benchmarks/bench_paths.py --path rows            (1 GPU: HBM roofline)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/bench_paths.py --path rows               (N GPUs: NVLink roofline)

paths: rows (sparse keyed pull / push of 128-float rows), dense (dense read = all-gather,
dense bupdate = reduce-scatter + prox-L1 handler), gather_gemm (all-gather of a sharded B fused
with the tcgen05 GEMM), ssp (commit + wait latency), allreduce (one-launch small all-reduce).

Timing: CUDA events, 3 warm-ups, median of the timed launches, a 256 MB buffer is rewritten
between launches to flush L2, max over ranks.  The roofline denominator is the measured copy
bandwidth of MEASURED_PEAKS.json ("of measured") for local bytes and 770 GB/s per direction for
bytes that cross NVLink."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--path", required=True, choices=["rows", "dense", "gather_gemm", "ssp", "allreduce"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true", help="smaller sizes (for ncu captures)")
    ap.add_argument("--table-rows", type=int, default=0, help="rows path: total table rows (default 4 M per rank)")
    ap.add_argument("--push-rows", type=int, default=0, help="rows path: rows pulled / pushed per rank")
    ap.add_argument("--sorted-ids", action="store_true", help="rows path: ascending ids instead of a random order")
    ap.add_argument("--kernel", default=None, choices=["1sm", "2sm"], help="GEMM kernel of gather_gemm")
    ap.add_argument("--gather-ctas", type=int, default=0, help="gather_gemm: CTAs that stage the peers' shards "
                    "(0: the operator's default)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lrank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lrank)
    dev = torch.device("cuda", lrank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peaks = json.load(open(os.path.join(root, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(root, "MEASURED_PEAKS.json")) else {}
    hbm = peaks.get("hbm_gbs", 6650.0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timeit(fn, pre=None):
        ts = []
        for it in range(3 + args.iters):
            if pre:
                pre()
            flush.zero_()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        ms = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    out = {"path": args.path, "n_gpus": world}
    if args.path == "rows":
        from paracel_b200.ps.tables import RowTable
        rows = (1 << 20) if args.small else (1 << 22)
        total_rows = args.table_rows or rows * world
        t = RowTable(total_rows, 128, torch.float32)
        t.shard.normal_()
        n = args.push_rows or rows // 2
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        ids = torch.randperm(total_rows, device=dev, generator=g)[:n].contiguous()
        if args.sorted_ids:
            ids = torch.sort(ids).values.contiguous()
        cur = torch.empty(n, 128, device=dev)
        old = torch.empty_like(cur)
        wgt = torch.rand(n, device=dev)
        barrier()
        ms_pull = timeit(lambda: t.pull(ids, cur, old))
        cur += 1.0
        ms_push = timeit(lambda: t.push(ids, cur, old, wgt, refresh_old=False))

        row_b = 512.0
        remote = (world - 1) / world
        out.update({
            "rows": n, "pull_ms": ms_pull, "push_ms": ms_push,
            "pull_GBps_algorithmic": 3 * n * row_b / ms_pull / 1e6,     # 1 read + 2 writes
            "push_GBps_algorithmic": 3 * n * row_b / ms_push / 1e6,     # 2 reads + 1 reduction
            "pull_frac_hbm_of_measured": 3 * n * row_b / ms_pull / 1e6 / hbm,
            "push_frac_hbm_of_measured": 3 * n * row_b / ms_push / 1e6 / hbm,
            "pull_nvlink_GBps": remote * n * row_b / ms_pull / 1e6,
            "push_nvlink_GBps": remote * n * row_b / ms_push / 1e6,
            "pull_frac_nvlink_770": remote * n * row_b / ms_pull / 1e6 / NVLINK_GBS if world > 1 else None,
            "push_frac_nvlink_770": remote * n * row_b / ms_push / 1e6 / NVLINK_GBS if world > 1 else None})
        barrier()
        t.free()
    elif args.path == "dense":
        from paracel_b200.ps.tables import DenseTable
        L = (1 << 24) if args.small else (1 << 26)
        t = DenseTable(L, handler="prox_l1", lr=0.1, lam=1e-3)
        t.write(torch.randn(L, device=dev))
        barrier()
        ms_read = timeit(lambda: t.read())

        def upd():
            t.delta().normal_() if False else None
            t.bupdate()
        t.delta_buf.local.normal_()
        ms_bup = timeit(upd)
        torch.cuda.synchronize()
        t.check()
        S = t.S
        remote = (world - 1) / world
        out.update({
            "L": L, "read_ms": ms_read, "bupdate_ms": ms_bup,
            "read_GBps_algorithmic": 2 * L * 4 / ms_read / 1e6,
            "read_frac_hbm_of_measured": 2 * L * 4 / ms_read / 1e6 / hbm,
            "read_nvlink_GBps": remote * L * 4 / ms_read / 1e6,
            "read_frac_nvlink_770": remote * L * 4 / ms_read / 1e6 / NVLINK_GBS if world > 1 else None,
            # owner reads world slices of S floats and rewrites its shard
            "bupdate_GBps_algorithmic": (world + 2) * S * 4 / ms_bup / 1e6,
            "bupdate_frac_hbm_of_measured": (world + 2) * S * 4 / ms_bup / 1e6 / hbm,
            "bupdate_nvlink_GBps": (world - 1) * S * 4 / ms_bup / 1e6,
            "bupdate_frac_nvlink_770": (world - 1) * S * 4 / ms_bup / 1e6 / NVLINK_GBS if world > 1 else None})
        barrier()
        t.free()
    elif args.path == "gather_gemm":
        from paracel_b200.ops.gemm import DenseReadGemm
        N, K, M = (4096, 256, 32768) if args.small else (16384, 512, 65536)
        op = DenseReadGemm(N, K, kernel=args.kernel, **({"gather_ctas": args.gather_ctas} if args.gather_ctas else {}))
        op.shard.normal_()
        A = torch.randn(M, K, device=dev)
        C = torch.empty(M, N, device=dev)
        barrier()
        ms = timeit(lambda: op(A, out=C))
        op.check()
        flops = 2.0 * M * N * K
        gathered = (world - 1) / world * N * K * 4
        t_flops = flops / (peaks.get("bf16_tflops", 1590.0) / 2 * 1e12) * 1e3   # tf32 = half the bf16 rate
        t_link = gathered / (NVLINK_GBS * 1e9) * 1e3
        out.update({"kernel": args.kernel or "default", "gather_ctas": op.gather_ctas, "M": M, "N": N, "K": K, "ms": ms, "tflops": flops / ms / 1e9,
                    "gathered_MB": gathered / 1e6, "roofline_ms": max(t_flops, t_link),
                    "frac_of_roofline": max(t_flops, t_link) / ms,
                    "roofline_note": "max(FLOPs / (measured bf16 burst / 2), gathered bytes / 770 GB/s)"})
        barrier()
        op.free()
    elif args.path == "ssp":
        from paracel_b200.parallel.ssp_device import DeviceSspClock
        c = DeviceSspClock(2, 1 << 30)
        barrier()

        def step():
            c.wait()
            c.commit()
        ms = timeit(step)
        c.check()
        out.update({"commit_plus_wait_us": ms * 1e3})
        barrier()
        c.free()
    else:
        from paracel_b200.ops.misc import DeviceAllReduce
        ar = DeviceAllReduce()
        x = torch.ones(2, dtype=torch.float64, device=dev)
        y = torch.empty_like(x)
        barrier()
        ms = timeit(lambda: ar(x, y))
        ar.check()
        z = torch.ones(2, dtype=torch.float64, device=dev)
        ms_nccl = timeit(lambda: dist.all_reduce(z)) if world > 1 else None
        out.update({"one_launch_allreduce_us": ms * 1e3, "nccl_allreduce_us": ms_nccl * 1e3 if ms_nccl else None})
        barrier()
        ar.free()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
