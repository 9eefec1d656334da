"""k-means on GPUs (device path of alg/clustering/kmeans/kmeans.hpp:40-200).

The centres (k x d) are a parameter range-sharded by rows over the ranks.  One round:

    assignment  = all-gather of the centre shards fused with the tcgen05 GEMM X . C^T and a
                  row-wise arg-min epilogue                              (DenseReadGemm)
    local sums  = per-cluster sums and counts of the local rows          (kmeans_accumulate)
    new centres = reduce-scatter(add) of [sums | counts] fused with the add handler, then the
                  owners divide and store their rows                     (DenseTable)

which is the reference's read("clusters_{rd-1}") / all-reduce of counts / bupdate of
``local_sum / global_count`` with the add handler."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.gemm import DenseReadGemm
from ..ops.misc import kmeans_accumulate
from ..ps.tables import DenseTable


class KMeansGpu:
    def __init__(self, kclusters: int, dim: int, group=None, device=None, precise: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k, self.d = int(kclusters), int(dim)
        self.dp = (self.d + 3) // 4 * 4                   # GEMM needs K % 4 == 0
        # precise: operands are split into tf32-exact high and low parts along K (3xTF32), so
        # that near ties are assigned as in fp32 arithmetic; the shard then holds [hi | lo | hi]
        self.precise = precise
        self.kw = 3 * self.dp if precise else self.dp
        self.centres = DenseReadGemm(self.k, self.kw, group, device)
        self.acc = DenseTable(self.k * self.dp + self.k, group, device, handler="add")
        self.device = self.centres.device

    def load(self, X: torch.Tensor, init_centres: Optional[torch.Tensor] = None):
        """Local rows X [n, d]; ``init_centres`` (k x d, identical on every rank) defaults to the
        first k rows of rank 0, as in the reference (kmeans.hpp:79-93)."""
        dev = self.device
        n = X.shape[0]
        self.X = torch.zeros(n, self.dp, device=dev)
        self.X[:, : self.d] = X.to(dev, torch.float32)
        if init_centres is None:
            init_centres = self.X[: self.k, : self.d].clone()
            if self.world > 1:
                dist.broadcast(init_centres, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                               group=self.group)
        lo, hi = self.centres.local_rows()
        self.c_local = torch.zeros(self.centres.rps, self.dp, device=dev)   # fp32 master of my rows
        if hi > lo:
            self.c_local[: hi - lo, : self.d] = init_centres[lo:hi].to(dev, torch.float32)
        self._publish_centres()
        if self.precise:
            from ..ops.gemm import split3
            self.Xg = split3(self.X, False)
        else:
            self.Xg = self.X
        self.assign = torch.zeros(n, dtype=torch.int32, device=dev)
        self.acc.write(torch.zeros(self.acc.L, device=dev))
        self._barrier()

    def _barrier(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def _publish_centres(self):
        if self.precise:
            from ..ops.gemm import split3
            self.centres.shard.copy_(split3(self.c_local, True))
        else:
            self.centres.shard.copy_(self.c_local)

    def round(self):
        lo, hi = self.centres.local_rows()
        # |c|^2 of every centre: owners know their rows, the rest comes with the gathered copy of
        # the previous call; computed from a small all-gather to stay exact in the first round
        shard_norm = (self.c_local * self.c_local).sum(1)
        if self.world > 1:
            parts = [torch.empty_like(shard_norm) for _ in range(self.world)]
            dist.all_gather(parts, shard_norm, group=self.group)
            bnorm = torch.cat(parts)[: self.k].contiguous()
        else:
            bnorm = shard_norm[: self.k].contiguous()
        _, arg = self.centres(self.Xg, argmin_bnorm=bnorm)
        self.assign = arg
        delta = self.acc.delta()
        delta.zero_()
        sums = delta[: self.k * self.dp].view(self.k, self.dp)
        counts = delta[self.k * self.dp:]
        kmeans_accumulate(self.X, arg, sums, counts)
        # the accumulator table holds only this round's sums: reset the owner shards, then reduce
        self.acc.shard.zero_()
        self.acc.bupdate(handler="add")
        tot = self.acc.read()
        gs = tot[: self.k * self.dp].view(self.k, self.dp)
        gc = tot[self.k * self.dp:]
        self._barrier()   # everybody has consumed the old centres before the owners overwrite them
        if hi > lo:
            cnt = gc[lo:hi].clamp(min=1.0)[:, None]
            new = gs[lo:hi] / cnt
            keep = (gc[lo:hi] == 0)[:, None]          # an empty cluster keeps its centre
            self.c_local[: hi - lo] = torch.where(keep, self.c_local[: hi - lo], new)
        self._publish_centres()
        self._barrier()

    def fit(self, rounds: int):
        for _ in range(rounds):
            self.round()
        self.centres.check()
        self.acc.check()

    def cluster_centres(self) -> torch.Tensor:
        """All k centres (k x d), gathered."""
        sh = self.c_local
        if self.world > 1:
            parts = [torch.empty_like(sh) for _ in range(self.world)]
            dist.all_gather(parts, sh.contiguous(), group=self.group)
            sh = torch.cat(parts)
        return sh[: self.k, : self.d].clone()

    def free(self):
        self._barrier()
        self.centres.free()
        self.acc.free()
