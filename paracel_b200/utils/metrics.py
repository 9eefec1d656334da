"""Run metrics, logging and phase timing.

The reference only prints progress lines and keeps wall-clock accumulators in LDA
(alg/topic_model/gLDA.hpp:409-444) plus the launcher's command log.  Here:

* ``get_logger``     Python logging with a ``[rank r]`` prefix;
* ``MetricsLogger``  one JSON object per line in ``metrics.jsonl`` (round, loss, throughput,
                     bytes pulled / pushed, staleness, wait time, ...);
* ``PhaseTimer``     named phases timed with CUDA events on the current stream (or
                     ``perf_counter`` without a GPU), optional NVTX ranges, summarised as a
                     per-rank JSON trace; ``max_over_ranks`` reduces a duration the way the
                     benchmarks report it."""
from __future__ import annotations

import json
import logging
import os
import time
from contextlib import contextmanager
from typing import Any, Dict, List, Optional


def get_logger(name: str = "paracel", rank: Optional[int] = None, level: int = logging.INFO) -> logging.Logger:
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    lg = logging.getLogger(f"{name}.r{rank}")
    if not lg.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(f"%(asctime)s [rank {rank}] %(levelname)s %(message)s"))
        lg.addHandler(h)
        lg.propagate = False
    lg.setLevel(level)
    return lg


class MetricsLogger:
    def __init__(self, path: str, rank: int = 0, only_rank0: bool = True):
        self.enabled = (rank == 0) or not only_rank0
        self.rank = rank
        self.path = path
        if self.enabled:
            d = os.path.dirname(path)
            if d:
                os.makedirs(d, exist_ok=True)
            self.f = open(path, "a")

    def log(self, **kv: Any) -> None:
        if not self.enabled:
            return
        kv.setdefault("ts", time.time())
        kv.setdefault("rank", self.rank)
        self.f.write(json.dumps(kv) + "\n")
        self.f.flush()

    def close(self) -> None:
        if self.enabled:
            self.f.close()

    @staticmethod
    def read(path: str) -> List[Dict[str, Any]]:
        with open(path) as f:
            return [json.loads(l) for l in f if l.strip()]


class PhaseTimer:
    def __init__(self, use_cuda: Optional[bool] = None, nvtx: bool = False):
        import torch
        self.torch = torch
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.nvtx = nvtx and self.cuda
        self.events: List[tuple] = []
        self.cpu: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}

    @contextmanager
    def phase(self, name: str):
        if self.cuda:
            e0 = self.torch.cuda.Event(enable_timing=True)
            e1 = self.torch.cuda.Event(enable_timing=True)
            if self.nvtx:
                self.torch.cuda.nvtx.range_push(name)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                if self.nvtx:
                    self.torch.cuda.nvtx.range_pop()
                self.events.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self.cpu[name] = self.cpu.get(name, 0.0) + (time.perf_counter() - t0) * 1e3
                self.counts[name] = self.counts.get(name, 0) + 1

    def summary(self) -> Dict[str, Dict[str, float]]:
        """{phase: {ms, count}}; synchronises the device once."""
        out: Dict[str, Dict[str, float]] = {k: {"ms": v, "count": self.counts[k]} for k, v in self.cpu.items()}
        if self.cuda and self.events:
            self.torch.cuda.synchronize()
            for name, e0, e1 in self.events:
                d = out.setdefault(name, {"ms": 0.0, "count": 0})
                d["ms"] += e0.elapsed_time(e1)
                d["count"] += 1
            self.events = []
        return out

    def dump(self, path: str, rank: int = 0) -> None:
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(path, "w") as f:
            json.dump({"rank": rank, "phases": self.summary()}, f, indent=1)


def max_over_ranks(ms: float, group=None) -> float:
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ms
    dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) != "gloo" else "cpu"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
