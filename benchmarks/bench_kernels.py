#!/usr/bin/env python
"""Micro-benchmarks of the single-GPU algorithm kernels against stock PyTorch ops doing the same
job: batched ALS solve, k-means accumulate, Gram matrix, device ball-tree search, dense LR gradient,
the CSR products of the SVD, blockwise similarity with top-k.  CUDA events, 3 warm-ups, L2 flushed
between timed launches, one JSON line per kernel.

    python benchmarks/bench_kernels.py [--kernel als|kmeans|gram|balltree|dense_grad|spmm|sim_topk|all]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch


def timeit(fn, flush, iters=5, warmup=3):
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


def bench_als(flush):
    from paracel_b200.ops.als import als_solve
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    n_users, n_items, k, per_user = 200_000, 100_000, 128, 100
    H = torch.randn(n_items, k, device=dev, generator=g) * 0.1
    ptr = torch.arange(0, n_users * per_user + 1, per_user, device=dev, dtype=torch.int64)
    idx = torch.randint(0, n_items, (n_users * per_user,), device=dev, generator=g, dtype=torch.int32)
    r = torch.rand(n_users * per_user, device=dev, generator=g) * 4 + 1
    ms = timeit(lambda: als_solve(ptr, idx, r, H, 0.1), flush)
    # stock ops on a slice (the batched Gram build needs n_users x per_user x k floats)
    nb = 20_000

    def torch_ref():
        Hu = H[idx[: nb * per_user].long()].view(nb, per_user, k)
        A = Hu.transpose(1, 2) @ Hu + 0.1 * torch.eye(k, device=dev)
        b = (Hu * r[: nb * per_user].view(nb, per_user, 1)).sum(1)
        return torch.linalg.solve(A, b)
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_ref = timeit(torch_ref, flush) * (n_users / nb)
    flops = n_users * (2.0 * per_user * k * k + k ** 3 / 3.0 + 2 * k * k)
    return {"kernel": "als_solve", "users": n_users, "ratings_per_user": per_user, "k": k, "ms": ms,
            "systems_per_s": n_users / ms * 1e3, "tflops_fp32": flops / ms / 1e9,
            "torch_gather_bmm_solve_ms_scaled": ms_ref, "speedup": ms_ref / ms}


def bench_kmeans(flush):
    from paracel_b200.ops.misc import kmeans_accumulate
    dev = "cuda"
    n, d, k = 4_000_000, 128, 1024
    X = torch.randn(n, d, device=dev)
    assign = torch.randint(0, k, (n,), device=dev, dtype=torch.int32)
    sums = torch.zeros(k, d, device=dev)
    counts = torch.zeros(k, device=dev)

    def ours():
        sums.zero_(); counts.zero_()
        kmeans_accumulate(X, assign, sums, counts)

    def ref():
        sums.zero_(); counts.zero_()
        sums.index_add_(0, assign.long(), X)
        counts.index_add_(0, assign.long(), torch.ones(n, device=dev))
    ms, ms_ref = timeit(ours, flush), timeit(ref, flush)
    return {"kernel": "kmeans_accumulate", "n": n, "d": d, "k": k, "ms": ms, "GBps": n * d * 4 / ms / 1e6,
            "torch_index_add_ms": ms_ref, "speedup": ms_ref / ms}


def bench_gram(flush):
    from paracel_b200.ops.misc import gram
    dev = "cuda"
    n, k = 8_000_000, 64
    H = torch.randn(n, k, device=dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    ms, ms_ref = timeit(lambda: gram(H), flush), timeit(lambda: H.T @ H, flush)
    return {"kernel": "gram", "n": n, "k": k, "ms": ms, "GBps": n * k * 4 / ms / 1e6,
            "torch_fp32_matmul_ms": ms_ref, "speedup": ms_ref / ms}


def bench_balltree(flush):
    import numpy as np
    from paracel_b200.tool.balltree import DeviceBalltree, PyBalltree
    rng = np.random.default_rng(0)
    # clustered items: branch and bound can prune
    centres = rng.standard_normal((200, 64)) * 4
    items = (centres[rng.integers(0, 200, 200_000)] + rng.standard_normal((200_000, 64)) * 0.3)
    tree = PyBalltree(items)
    tree.build()
    dt = DeviceBalltree(tree)
    Q = torch.as_tensor((centres[rng.integers(0, 200, 8192)] + rng.standard_normal((8192, 64)) * 0.3)
                        .astype(np.float32), device="cuda")
    ms = timeit(lambda: dt.search(Q, 10), flush)
    X = dt.items

    def brute():
        return torch.topk(Q @ X.T, 10, dim=1)
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_ref = timeit(brute, flush)
    _, _, vis = dt.search(Q, 10)
    return {"kernel": "balltree_search", "items": 200_000, "dim": 64, "queries": 8192, "k": 10, "ms": ms,
            "queries_per_s": 8192 / ms * 1e3, "mean_balls_opened": float(vis.float().mean().item()),
            "nodes": tree.node_count, "torch_matmul_topk_ms": ms_ref}


def bench_dense_grad(flush):
    from paracel_b200.ops.linear import DenseGrad
    dev = torch.device("cuda")
    n, d = 2_000_000, 512
    X = torch.randn(n, d, device=dev)
    y = (torch.rand(n, device=dev) > 0.5).float()
    th = torch.randn(d, device=dev) * 0.1
    g = torch.empty(d, device=dev)
    dg = DenseGrad(d, dev)
    ms = timeit(lambda: dg(X, y, th, g), flush)

    def ref():
        h = torch.sigmoid(X @ th)
        return X.T @ (y - h)
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_ref = timeit(ref, flush)
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    gbs = n * d * 4 / ms / 1e6
    return {"kernel": "lr_dense_grad", "n": n, "d": d, "ms": ms, "GBps": gbs,
            "frac_hbm_of_measured": gbs / peaks.get("hbm_gbs", 6650.0), "torch_two_matvec_ms": ms_ref,
            "speedup": ms_ref / ms}


def bench_spmm(flush):
    """A.H and A^T.W for a CSR matrix with 64-wide dense factors against torch.sparse.mm."""
    from paracel_b200.ops.svd import spmm_csr, spmm_csr_t
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(2)
    m, n, per_row, K = 2_000_000, 500_000, 40, 64
    cols = torch.randint(0, n, (m * per_row,), device=dev, generator=g, dtype=torch.int32)
    vals = torch.rand(m * per_row, device=dev, generator=g)
    ptr = torch.arange(0, m * per_row + 1, per_row, device=dev, dtype=torch.int64)
    H = torch.randn(n, K, device=dev, generator=g)
    W = torch.randn(m, K, device=dev, generator=g)
    out_w = torch.empty(m, K, device=dev)
    out_h = torch.zeros(n, K, device=dev)
    ms = timeit(lambda: spmm_csr(ptr, cols, vals, H, out_w), flush)

    def ours_t():
        out_h.zero_()
        spmm_csr_t(ptr, cols, vals, W, out_h)
    ms_t = timeit(ours_t, flush)
    A = torch.sparse_csr_tensor(ptr, cols.long(), vals, (m, n))
    At = A.to_sparse_coo().t().coalesce().to_sparse_csr()
    ms_ref = timeit(lambda: torch.sparse.mm(A, H), flush)
    ms_ref_t = timeit(lambda: torch.sparse.mm(At, W), flush)
    nnz = m * per_row
    return {"kernel": "spmm_csr / spmm_csr_t", "rows": m, "cols": n, "nnz": nnz, "K": K, "ms": ms, "ms_t": ms_t,
            "gflops": 2.0 * nnz * K / ms / 1e6, "gflops_t": 2.0 * nnz * K / ms_t / 1e6,
            "torch_sparse_mm_ms": ms_ref, "torch_sparse_mm_t_ms_pretransposed": ms_ref_t,
            "speedup": ms_ref / ms, "speedup_t": ms_ref_t / ms_t}


def bench_sim_topk(flush):
    """Similarity of 16 k rows against 131 k rows (dim 128) with a running top-20: the 3xTF32
    tcgen05 GEMM + top-k kernel against torch.matmul (fp32) + torch.topk on the same tiles."""
    from paracel_b200.ops.gemm import split3
    from paracel_b200.ops.misc import RunningTopK
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(3)
    ma, nb, d, k = 16384, 131072, 128, 20
    A = torch.nn.functional.normalize(torch.randn(ma, d, device=dev, generator=g))
    B = torch.nn.functional.normalize(torch.randn(nb, d, device=dev, generator=g))
    ids_a = torch.arange(ma, device=dev) + 10_000_000
    ids_b = torch.arange(nb, device=dev)
    A3, B3 = split3(A, False), split3(B, True)
    S = torch.empty(ma, nb, device=dev)

    def ours():
        from paracel_b200.ops.gemm import _launch
        _launch(A3, B3, S, 0, None, None, None)
        t = RunningTopK(ids_a, k, 0.0)
        t.update(S, ids_b)
        return t
    torch.backends.cuda.matmul.allow_tf32 = False

    def ref():
        return torch.topk(A @ B.T, k, dim=1)
    ms, ms_ref = timeit(ours, flush), timeit(ref, flush)
    return {"kernel": "similarity 3xTF32 GEMM + top-k", "rows_a": ma, "rows_b": nb, "dim": d, "k": k, "ms": ms,
            "tflops_fp32_equiv": 2.0 * ma * nb * d / ms / 1e9, "torch_fp32_matmul_topk_ms": ms_ref,
            "speedup": ms_ref / ms}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", choices=["all", "als", "kmeans", "gram", "balltree", "dense_grad", "spmm",
                                                         "sim_topk"])
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = {"als": bench_als, "kmeans": bench_kmeans, "gram": bench_gram, "balltree": bench_balltree,
             "dense_grad": bench_dense_grad, "spmm": bench_spmm, "sim_topk": bench_sim_topk}
    for name, fn in table.items():
        if args.kernel in ("all", name):
            print(json.dumps(fn(flush)))


if __name__ == "__main__":
    main()
