#!/usr/bin/env python
"""Benchmarks of the remaining synthetic configurations (the flagship MF-SGD one is bench.py):

    lr_cpu    logistic regression, SGD, 2 workers + 1 parameter server on CPU, 20,000 x 100 dense,
              lr 0.01, 10 rounds, SSP staleness 1 (plumbing, no GPU)           -> samples/s
    l1lr      sparse L1 logistic regression, 50 M x 2^24 hashed features, 40 nnz/row Zipf(1.05),
              proximal-L1 handler, lambda 1e-6                                 -> samples/s
    lda       collapsed Gibbs LDA, 1 M docs, V 100 k Zipf(1.07), Poisson(200) tokens, K 1024,
              alpha 50/K, beta 0.01, SSP 2                                      -> tokens/s
    pagerank  R-MAT scale 26 (edge factor 16, a .57 b .19 c .19), d 0.85, 20 iterations
                                                                                -> edges/s per iteration

    python benchmarks/bench_configs.py --config l1lr [--scale 0.1] [--impl ours|nccl_torch]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/bench_configs.py --config pagerank --scale 0.05

``--scale`` shrinks the data size (1.0 = the full configuration).  Timing: CUDA events around
the timed steps after warm-up, barrier + synchronize on both sides, max over ranks.  Inputs are
larger than L2 at any scale >= 0.05.  Rank 0 prints one JSON line."""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def lr_cpu(args):
    import tempfile
    import numpy as np
    from paracel_b200.launch.local import LocalJob
    from paracel_b200.testing import cpu_workers as W
    rng = np.random.default_rng(0)
    n, d = 20000, 100
    X = rng.standard_normal((n, d))
    w = rng.standard_normal(d)
    y = (rng.random(n) < 1 / (1 + np.exp(-X @ w))).astype(float)
    tmp = tempfile.mkdtemp()
    inp = os.path.join(tmp, "train.csv")
    np.savetxt(inp, np.concatenate([X, y[:, None]], 1), delimiter=",", fmt="%.6f")
    res = LocalJob(2, 1).run(W.run_lr, (inp, os.path.join(tmp, "out"), "ipm", True, 10), timeout_s=600)
    sec = max(r["seconds"] for r in res)
    learn = max(r["seconds_learn"] for r in res)
    print(json.dumps({"config": "lr_cpu", "metric": "samples/s (LR, CPU plumbing)", "value": n * 10 / learn,
                      "seconds_10_rounds": learn, "seconds_load_and_parse": max(r["seconds_load"] for r in res),
                      "samples_per_s_including_load": n * 10 / sec, "final_logloss": res[0]["loss"],
                      "workers": 2, "servers": 1, "ssp_staleness": 1,
                      "note": "value counts the 10 learning rounds (pull, SGD pass, push, commit); "
                              "loading and parsing the CSV is reported separately"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["lr_cpu", "l1lr", "lda", "pagerank"])
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl_torch"])
    ap.add_argument("--steps", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-scramble", action="store_true",
                    help="pagerank: keep the raw R-MAT vertex labels (equal id ranges are then unbalanced)")
    args = ap.parse_args()
    if args.config == "lr_cpu":
        return lr_cpu(args)

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lrank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lrank)
    dev = torch.device("cuda", lrank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    from paracel_b200.ops import _lib
    from paracel_b200.utils import synth
    from paracel_b200.utils.clocks import ClockSampler
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    hbm = peaks.get("hbm_gbs", 6650.0)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        sampler = ClockSampler(lrank).start() if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launches()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        barrier()
        clocks = sampler.stop() if sampler else None
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, _lib.launches() - l0, clocks

    out = {"config": args.config, "impl": args.impl, "n_gpus": world, "scale": args.scale, "dtype": "fp32",
           "data": "synthetic, seeded"}
    t_setup = time.time()
    if args.config == "l1lr":
        n_total = int(50_000_000 * args.scale)
        F, k = 1 << 24, 40
        st = synth.SparseLrStream(n_total, F, k, 1.05, seed=7, device=dev)
        cols, ys = [], []
        for c in range(st.nchunks()):
            if c % world != rank:
                continue
            cc, yy = st.chunk_at(c)
            cols.append(cc)
            ys.append(yy)
        cols, y = torch.cat(cols), torch.cat(ys)
        n_local = y.numel()
        row_ptr = torch.arange(0, n_local * k + 1, k, device=dev, dtype=torch.int64)
        nbatch = 8
        steps = args.steps or nbatch
        if args.impl == "ours":
            from paracel_b200.models.linear_gpu import SparseLinearGpu
            m = SparseLinearGpu(F, eta=0.5, lam=1e-6, nbatch=nbatch, device=dev)
            m.load(row_ptr, cols, y)
            step = m.step
        else:
            from paracel_b200.baselines.nccl_torch import SparseLinearNcclTorch
            m = SparseLinearNcclTorch(F, eta=0.5, lam=1e-6, nbatch=nbatch, device=dev)
            m.load(row_ptr, cols, y)
            step = m.step
        ms, launches, clocks = timed(step, steps, args.warmup)
        rows_per_step = n_total / nbatch
        out.update({"metric": "samples/s (sparse L1-LR)", "value": rows_per_step / (ms * 1e-3),
                    "ms_per_step": ms, "samples_per_step": rows_per_step, "loss": m.mean_loss(),
                    "nnz_w": m.nnz_weights(), "gpu_launches": launches, "clocks": clocks,
                    # algorithmic bytes per step and GPU: indices read twice, theta gathered, g scattered,
                    # plus the dense table read / zero / reduce (4 x 64 MiB)
                    "hbm_fraction_of_measured": ((rows_per_step / world) * k * 4 * 2 + 5 * F * 4)
                    / (ms * 1e-3) / 1e9 / hbm})
    elif args.config == "lda":
        n_docs = int(1_000_000 * args.scale)
        V, K = 100_000, 1024
        d0, d1 = rank * n_docs // world, (rank + 1) * n_docs // world
        ptr, words = synth.lda_corpus_chunk(d1 - d0, V, 1.07, 200.0, seed=100 + rank, device=dev)
        nbatch = 8
        steps = args.steps or nbatch
        if args.impl == "ours":
            from paracel_b200.models.lda_gpu import LdaGibbsGpu
            m = LdaGibbsGpu(V, K, None, 0.01, iters=1000, nbatch=nbatch, staleness=2, device=dev)
            m.load_docs(ptr, words)
            step = m.step
        else:
            from paracel_b200.baselines.nccl_torch import LdaNcclTorch
            m = LdaNcclTorch(V, K, None, 0.01, nbatch=nbatch, device=dev)
            m.load_docs(ptr, words)
            step = m.step
        ms, launches, clocks = timed(step, steps, args.warmup)
        tok = torch.tensor([words.numel()], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(tok)
        tokens_per_step = tok.item() / nbatch
        ll = m.iteration(with_loglik=True) if args.impl == "ours" else None
        out.update({"metric": "tokens/s (LDA Gibbs)", "value": tokens_per_step / (ms * 1e-3), "ms_per_step": ms,
                    "tokens_per_step": tokens_per_step, "loglik_per_token": (ll / tok.item()) if ll else None,
                    "gpu_launches": launches, "clocks": clocks})
    else:
        scale_log = 26 + int(round(__import__("math").log2(max(args.scale, 1e-9))))
        n = 1 << scale_log
        m_edges = 16 * n
        from paracel_b200.models.pagerank_gpu import PageRankGpu
        if args.impl == "ours":
            pr = PageRankGpu(n, 0.85, device=dev)
        else:
            from paracel_b200.baselines.nccl_torch import PageRankNcclTorch
            pr = PageRankNcclTorch(n, 0.85, device=dev)
        srcs, dsts = [], []
        chunk = 1 << 26
        for c in range((m_edges + chunk - 1) // chunk):
            mm = min(chunk, m_edges - c * chunk)
            s, d = synth.rmat_edges_chunk(scale_log, mm, 0.57, 0.19, 0.19, seed=500 + c, device=dev)
            if not args.no_scramble:   # balanced ownership of equal id ranges (labels are arbitrary)
                s = synth.scramble_vertex_blocks(s, scale_log)
                d = synth.scramble_vertex_blocks(d, scale_log)
            keep = pr.owner_of(d) == rank
            srcs.append(s[keep].to(torch.int32))
            dsts.append(d[keep].to(torch.int32))
        src, dst = torch.cat(srcs).long(), torch.cat(dsts).long()
        del srcs, dsts
        pr.load_edges(src, dst)
        del src, dst
        torch.cuda.empty_cache()
        steps = args.steps or 20
        ms, launches, clocks = timed(pr.step, steps, args.warmup)
        e_local = torch.tensor([pr.n_edges_local], dtype=torch.int64, device=dev)
        emax = e_local.clone()
        if world > 1:
            dist.all_reduce(e_local)
            dist.all_reduce(emax, op=dist.ReduceOp.MAX)
        out.update({"metric": "edges/s per iteration (PageRank)", "value": e_local.item() / (ms * 1e-3),
                    "ms_per_iteration": ms, "vertices": n, "edges": int(e_local.item()),
                    "edges_max_rank": int(emax.item()), "gpu_launches": launches, "clocks": clocks,
                    # indices (4 B) + one 32-byte sector per random rank read, per edge
                    "hbm_fraction_of_measured": (emax.item() * 36 + 3 * n * 4) / (ms * 1e-3) / 1e9 / hbm})
    out["setup_s"] = time.time() - t_setup
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
