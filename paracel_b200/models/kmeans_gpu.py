"""k-means on GPUs (device path of alg/clustering/kmeans/kmeans.hpp:40-200).

``KMeansGpu`` is a ``paralg`` subclass on the device backend.  The centres (k x d) are the
matrix key ``clusters``, sharded by rows over the ranks; their squared norms the dense key
``cluster_norms``; the per-round sums the dense key ``cluster_sums``.  One round:

    norms       = paracel_read("cluster_norms"): waits (bounded, on flags in peer memory) until
                  every owner has published its new rows
    assignment  = paracel_read_matmul("clusters", X, argmin_bnorm=norms): all-gather of the
                  centre shards fused with the tcgen05 GEMM X . C^T and a row-wise arg-min
    local sums  = per-cluster sums and counts of the local rows (kmeans_accumulate) written
                  into paracel_delta_buffer("cluster_sums")
    new centres = collective paracel_bupdate("cluster_sums", ..., "local_update_kmeans_clusters"):
                  reduce-scatter fused with the add handler; the owners then divide, store
                  their rows and norms and paracel_commit_write("cluster_norms")

which is the reference's read("clusters_{rd-1}") / all-reduce of counts / bupdate of
``local_sum / global_count`` with the add handler.  No host barrier and no NCCL call sits in
the round: a rank overwrites its centre rows only after every rank has published the delta
of the round (which follows its GEMM on the stream), and nobody reads new rows before the
owner's flag arrives."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.misc import kmeans_accumulate
from ..paralg import paralg


class KMeansGpu(paralg):
    def __init__(self, kclusters: int, dim: int, group=None, device=None, precise: bool = True,
                 comm=None, hosts_dct_str=None, output: str = ""):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.group = group
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.k, self.d = int(kclusters), int(dim)
        self.dp = (self.d + 3) // 4 * 4                   # GEMM needs K % 4 == 0
        # precise: operands are split into tf32-exact high and low parts along K (3xTF32), so
        # that near ties are assigned as in fp32 arithmetic; the shard then holds [hi | lo | hi]
        self.precise = precise
        self.kw = 3 * self.dp if precise else self.dp
        self.centres = self.paracel_matrix_table("clusters", self.k, self.kw).table.g
        self.acc = self.paracel_dense_table("cluster_sums", self.k * self.dp + self.k,
                                            handler="local_update_kmeans_clusters").table
        # norms: owner r publishes the norms of its rows in slice r (slices padded to 16 bytes)
        self.rps4 = (self.centres.rps + 3) // 4 * 4
        self.norms = self.paracel_dense_table("cluster_norms", self.rps4 * self.world).table

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
        self.paracel_write("cluster_sums", torch.zeros(self.acc.L, device=dev))
        self._barrier()

    def _barrier(self):
        self.paracel_sync()

    def _publish_centres(self):
        """Owner side: store this rank's rows (split for 3xTF32 when precise) and their squared
        norms, then publish the epoch that readers of ``cluster_norms`` wait for."""
        shard = self.paracel_local_shard("clusters")
        if self.precise:
            from ..ops.gemm import split3
            shard.copy_(split3(self.c_local, True))
        else:
            shard.copy_(self.c_local)
        nsh = self.paracel_local_shard("cluster_norms")
        nsh.zero_()
        nsh[: self.centres.rps] = (self.c_local * self.c_local).sum(1)
        self.paracel_commit_write("cluster_norms")

    def round(self):
        lo, hi = self.centres.local_rows()
        rps = self.centres.rps
        nfull = self.paracel_read("cluster_norms")          # waits for every owner's new rows
        bnorm = nfull.view(self.world, self.rps4)[:, :rps].reshape(-1)[: self.k].contiguous()
        _, arg = self.paracel_read_matmul("clusters", self.Xg, argmin_bnorm=bnorm)
        self.assign = arg
        delta = self.paracel_delta_buffer("cluster_sums")
        delta.zero_()
        sums = delta[: self.k * self.dp].view(self.k, self.dp)
        counts = delta[self.k * self.dp:]
        kmeans_accumulate(self.X, arg, sums, counts)
        # the accumulator key holds only this round's sums: reset the owner shard, then reduce
        self.paracel_local_shard("cluster_sums").zero_()
        self.paracel_bupdate("cluster_sums", delta, "", "local_update_kmeans_clusters", collective=True)
        tot = self.paracel_read("cluster_sums")
        gs = tot[: self.k * self.dp].view(self.k, self.dp)
        gc = tot[self.k * self.dp:]
        if hi > lo:
            cnt = gc[lo:hi].clamp(min=1.0)[:, None]
            new = gs[lo:hi] / cnt
            keep = (gc[lo:hi] == 0)[:, None]          # an empty cluster keeps its centre
            self.c_local[: hi - lo] = torch.where(keep, self.c_local[: hi - lo], new)
        self._publish_centres()

    def checkpoint_extra(self):
        return {"c_local": self.c_local}

    def restore_extra(self, extra):
        self.c_local.copy_(extra["c_local"].to(self.device))
        self._publish_centres()

    def fit(self, rounds: int):
        for j in range(rounds):
            with self.phase("round"):
                self.round()
            self.log_metrics(round=j, rows=self.X.shape[0], clusters=self.k)
        self._barrier()
        self.paracel_check()

    def cluster_centres(self) -> torch.Tensor:
        """All k centres (k x d), gathered."""
        sh = self.c_local
        if self.world > 1:
            parts = [torch.empty_like(sh) for _ in range(self.world)]
            dist.all_gather(parts, sh.contiguous(), group=self.group)
            sh = torch.cat(parts)
        return sh[: self.k, : self.d].clone()

    def free(self):
        self.centres = self.acc = self.norms = None
        self.close()
