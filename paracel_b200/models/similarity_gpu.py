"""Cosine-similarity top-k on GPUs (device path of
alg/recommendation/similarity_dense/sim_dense.hpp:60-200 and of the ring over peers' blocks of
alg/recommendation/similarity_sparse/sim_sparse_row.hpp:98-107, 143-173).

``SimDenseGpu`` is a ``paralg`` subclass on the device backend.  Every rank normalises its block
of the B rows and stores it as its shard of the matrix key ``sim_block`` (rows of all ranks'
blocks in rank order, padded to a common block height).  A rank then compares its A rows against
ALL blocks with ``paracel_read_matmul("sim_block", A_chunk)``: the fused kernel stages the
peers' shards into local memory over NVLink in the ring order ``rank, rank+1, ...`` while the
tensor cores (3xTF32, fp32-level accuracy) already multiply the blocks that have arrived; a
top-k kernel then merges every similarity tile into the running per-row heaps (``ktop`` best
columns with similarity >= ``simbar`` and a different id).  Sparse rows are densified per
block when the column space is small enough (``SimSparseGpu``)."""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops.gemm import split3
from ..ops.misc import RunningTopK
from ..paralg import paralg


class SimDenseGpu(paralg):
    def __init__(self, dim: int, ktop: int = 20, simbar: float = 0.0, group=None, device=None,
                 comm=None, hosts_dct_str=None, output: str = "", chunk_rows: int = 16384):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.world, self.rank, self.group = self.get_worker_size(), self.get_worker_id(), group
        self.d, self.ktop, self.simbar = int(dim), int(ktop), float(simbar)
        self.dp = (self.d + 3) // 4 * 4
        self.chunk_rows = int(chunk_rows)
        self.result: Dict[int, List[Tuple[int, float]]] = {}

    @staticmethod
    def _normalise(X: torch.Tensor) -> torch.Tensor:
        n = X.norm(dim=1, keepdim=True)
        return X / torch.where(n > 0, n, torch.ones_like(n))

    def load(self, ids_a: torch.Tensor, A: torch.Tensor, ids_b: Optional[torch.Tensor] = None,
             B: Optional[torch.Tensor] = None):
        """This rank's rows of A (ids + features) and its block of B (default: the same rows)."""
        dev = self.device
        if B is None:
            ids_b, B = ids_a, A
        self.ids_a = ids_a.to(dev, torch.int64).contiguous()
        self.A = torch.zeros(A.shape[0], self.dp, device=dev)
        self.A[:, : self.d] = self._normalise(A.to(dev, torch.float32))
        nb = torch.tensor([B.shape[0]], dtype=torch.int64, device=dev)
        allnb = [nb.clone() for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(allnb, nb, group=self.group)
        counts = [int(x.item()) for x in allnb]
        self.rps = max(max(counts), 1)                    # common block height
        # ids of every row of the gathered matrix (-1 marks padding rows)
        mine = torch.full((self.rps,), -1, dtype=torch.int64, device=dev)
        mine[: B.shape[0]] = ids_b.to(dev, torch.int64)
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(parts, mine, group=self.group)
        else:
            parts = [mine]
        self.ids_b_all = torch.cat(parts).contiguous()
        self.tab = self.paracel_matrix_table("sim_block", self.rps * self.world, 3 * self.dp)
        Bn = torch.zeros(self.rps, self.dp, device=dev)
        Bn[: B.shape[0], : self.d] = self._normalise(B.to(dev, torch.float32))
        self.paracel_local_shard(self.tab).copy_(split3(Bn, True))
        self.paracel_sync()                               # every block is in place

    def solve(self):
        topk = RunningTopK(self.ids_a, self.ktop, self.simbar)
        m = self.A.shape[0]
        # padding rows carry id -1: give them the row's own id semantics by masking afterwards
        for r0 in range(0, m, self.chunk_rows):
            r1 = min(m, r0 + self.chunk_rows)
            S = self.paracel_read_matmul("sim_block", split3(self.A[r0:r1].contiguous(), False))
            S[:, self.ids_b_all < 0] = -3.0e38
            part = RunningTopK(self.ids_a[r0:r1], self.ktop, self.simbar)
            part.update(S, self.ids_b_all)
            topk.val[r0:r1], topk.idx[r0:r1] = part.val, part.idx
        self.paracel_sync()
        self.paracel_check()
        self.result = topk.result() if m else {}

    def dump_result(self, outdir: str = ""):
        from ..utils.dump import dump_dict_pairs
        outdir = outdir or self.output
        os.makedirs(outdir, exist_ok=True)
        dump_dict_pairs({k: v for k, v in self.result.items() if v},
                        os.path.join(outdir, f"result_{self.rank}"))
        self.paracel_sync()

    def free(self):
        self.close()


class SimSparseGpu(SimDenseGpu):
    """Row similarity of a sparse matrix (``row,col,val`` triples): rows are densified over the
    global column space (at most ``max_cols`` columns) and handled by the dense path; the
    reference normalises and compares the same rows with sparse dot products
    (sim_sparse_row.hpp:82-173)."""

    def __init__(self, n_cols: int, ktop: int = 20, sim_bar: float = 0.0, max_cols: int = 65536, **kw):
        if n_cols > max_cols:
            raise ValueError(f"{n_cols} columns exceed the densified limit of {max_cols}")
        super().__init__(n_cols, ktop, sim_bar, **kw)

    def load_triples(self, row_ids: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor):
        """``row_ids``: original ids of the local rows; ``rows`` index them; ``cols`` in [0, n_cols)."""
        dev = self.device
        X = torch.zeros(row_ids.numel(), self.d, device=dev)
        X.index_put_((rows.to(dev, torch.int64), cols.to(dev, torch.int64)), vals.to(dev, torch.float32),
                     accumulate=False)
        self.load(row_ids, X)
