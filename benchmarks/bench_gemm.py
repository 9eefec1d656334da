#!/usr/bin/env python
"""Micro-benchmark of the tcgen05 tf32 GEMM (A @ B.T) against cuBLAS tf32 and fp32
(torch.matmul).  CUDA events, warm-up, L2 flushed between timed launches.

    python benchmarks/bench_gemm.py --m 65536 --n 1024 --k 128
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch


def timeit(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--k", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--kernel", default="2sm", choices=["1sm", "2sm"],
                    help="1sm: one CTA per 128x128 tile; 2sm: CTA pairs on 256x256 / 256x512 items")
    args = ap.parse_args()
    from paracel_b200.ops.gemm import argmin_nt, check_status, gemm_nt
    dev = "cuda"
    A = torch.randn(args.m, args.k, device=dev)
    B = torch.randn(args.n, args.k, device=dev)
    C = torch.empty(args.m, args.n, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    flops = 2.0 * args.m * args.n * args.k
    out = {"m": args.m, "n": args.n, "k": args.k, "kernel": args.kernel}
    kn = args.kernel
    t = timeit(lambda: gemm_nt(A, B, out=C, kernel=kn), flush, args.iters)
    check_status()
    out["ours_tf32_ms"] = t
    out["ours_tf32_tflops"] = flops / t / 1e9
    t = timeit(lambda: gemm_nt(A, B, out=C, precise=True, kernel=kn), flush, args.iters)
    out["ours_3xtf32_ms"] = t
    t = timeit(lambda: argmin_nt(A, B, kernel=kn), flush, args.iters)
    out["ours_argmin_ms"] = t
    check_status()
    torch.backends.cuda.matmul.allow_tf32 = True
    t = timeit(lambda: torch.matmul(A, B.T, out=C), flush, args.iters)
    out["cublas_tf32_ms"] = t
    out["cublas_tf32_tflops"] = flops / t / 1e9
    torch.backends.cuda.matmul.allow_tf32 = False
    t = timeit(lambda: torch.matmul(A, B.T, out=C), flush, args.iters)
    out["cublas_fp32_ms"] = t
    bytes_moved = 4.0 * (args.m * args.k + args.n * args.k + args.m * args.n)
    out["algorithmic_GBps_ours"] = bytes_moved / out["ours_tf32_ms"] / 1e6
    print(json.dumps(out))


if __name__ == "__main__":
    main()
