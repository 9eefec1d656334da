"""Distributed load on the GPUs: placement of parsed triples on the rank grid, exchange,
id compaction and CSR build, all on device tensors.

The host loader (``loader.py`` / ``scheduler.py``) bins Python triples and ships them with a
gloo all-to-all; this module does the same job for tensors that are already on the device
(a parsed shard, a synthetic generator): one histogram kernel, one host exchange of the
count matrix, and one scatter kernel that stores every triple directly into the receive
arrays of its destination rank over NVLink (``csrc/cuda/loader.cu``).  Placement, grid
shapes per pattern and the renumbering rules are those of the reference
(include/load/scheduler.hpp:75-95 placement, 157-170 exchange, 172-343 index mapping):
ranks of one grid row share the row ids, ranks of one grid column share the column ids.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..parallel.symm import SymmBuffer
from ..utils.decomp import npfact2d, npfactx, npfacty


def grid_of(pattern: str, world: int) -> Tuple[int, int]:
    if pattern == "fsmap":
        return npfact2d(world)
    if pattern == "smap":
        return npfacty(world)
    return npfactx(world)


class DeviceExchange:
    def __init__(self, pattern: str = "fmap", group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.pattern = pattern
        self.npx, self.npy = grid_of(pattern, self.world)
        self.status = torch.zeros(4, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ placement
    def owner(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """Destination rank of every triple (plain tensor arithmetic; the oracle of the kernels)."""
        return (a % self.npx) * self.npy + (b % self.npy)

    def exchange(self, a: torch.Tensor, b: torch.Tensor, w: torch.Tensor):
        """All-to-all by owner.  ``a``, ``b`` int64 ids (non-negative), ``w`` fp32 weights of this
        rank's parsed triples; returns the triples this rank owns (order unspecified)."""
        _lib.check_cuda(a, torch.int64, "a")
        _lib.check_cuda(b, torch.int64, "b")
        _lib.check_cuda(w, torch.float32, "w")
        n = a.numel()
        assert b.numel() == n and w.numel() == n
        world = self.world
        counts = torch.zeros(world, dtype=torch.int64, device=self.device)
        _lib.call("pcl_partition_count", a, b, n, self.npx, self.npy, counts, _lib.stream_ptr())
        if world == 1:
            return a.clone(), b.clone(), w.clone()
        # count matrix C[src][dst]
        mat = torch.empty(world, world, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(mat, counts, group=self.group)
        mat_h = mat.cpu()
        recv_tot = mat_h.sum(0)                       # per destination
        cap = int(recv_tot.max().item())
        cap = max(2, (cap + 1) // 2 * 2)              # keeps the fp32 block 8-byte aligned
        # where this source rank's block starts in every destination
        base_h = torch.zeros(world, dtype=torch.int64)
        for d in range(world):
            base_h[d] = int(mat_h[: self.rank, d].sum().item())
        base = base_h.to(self.device)
        quota = mat_h[self.rank].contiguous().to(self.device)
        buf = SymmBuffer(2 * cap + cap // 2, torch.int64, self.group, self.device)
        cursor = torch.zeros(world, dtype=torch.int64, device=self.device)
        self._barrier()                               # every receive buffer exists
        _lib.call("pcl_partition_scatter", a, b, w, n, self.npx, self.npy, buf.ptr_table, cap, base, quota,
                  cursor, self.status, self.rank, _lib.stream_ptr())
        torch.cuda.synchronize(self.device)
        self._barrier()                               # every peer has finished storing
        self.check()
        m = int(recv_tot[self.rank].item())
        loc = buf.local
        ra = loc[:m].clone()
        rb = loc[cap:cap + m].clone()
        rw = loc[2 * cap:].view(torch.float32)[:m].clone()
        self._barrier()
        buf.free()
        return ra, rb, rw

    def _barrier(self):
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    def check(self):
        st = self.status.cpu()
        if int(st[0].item()) & 0xFFFFFFFF:
            self.status.zero_()
            raise RuntimeError(f"device exchange: destination block overrun (expected at most "
                               f"{int(st[2])} triples, cursor reached {int(st[3])})")

    # --------------------------------------------------------------- id compaction
    def _union_over(self, ids: torch.Tensor, color: int, colors) -> torch.Tensor:
        """Sorted union of ``ids`` over the ranks whose colour equals ``color``."""
        if self.world == 1:
            return ids
        n = torch.tensor([ids.numel()], dtype=torch.int64, device=self.device)
        sizes = torch.empty(self.world, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(sizes, n, group=self.group)
        sizes_h = sizes.cpu().tolist()
        mx = max(1, max(sizes_h))
        pad = torch.zeros(mx, dtype=torch.int64, device=self.device)
        pad[: ids.numel()] = ids
        allv = torch.empty(self.world * mx, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(allv, pad, group=self.group)
        parts = [allv[r * mx: r * mx + sizes_h[r]] for r in range(self.world) if colors[r] == color]
        return torch.unique(torch.cat(parts))

    def index_mapping(self, a: torch.Tensor, b: torch.Tensor):
        """Dense renumbering of the owned triples.  Returns (row index, column index, rm, cm):
        ``rm[i]`` is the original id of local row i (sorted ascending, shared by the ranks of this
        grid row), ``cm`` likewise for columns."""
        row_colors = [r // self.npy for r in range(self.world)]
        col_colors = [r % self.npy for r in range(self.world)]
        rm = self._union_over(torch.unique(a), row_colors[self.rank], row_colors)
        cm = self._union_over(torch.unique(b), col_colors[self.rank], col_colors)
        ri = torch.searchsorted(rm, a)
        ci = torch.searchsorted(cm, b)
        return ri, ci, rm, cm

    @staticmethod
    def to_csr(ri: torch.Tensor, ci: torch.Tensor, w: torch.Tensor, n_rows: int):
        """CSR (int64 offsets, int32 column indices, fp32 values) of renumbered triples, rows and
        the columns inside a row ascending."""
        n_cols = int(ci.max().item()) + 1 if ci.numel() else 1
        key = ri * n_cols + ci
        order = torch.argsort(key)
        counts = torch.bincount(ri, minlength=n_rows)
        rowptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=ri.device)
        torch.cumsum(counts, 0, out=rowptr[1:])
        return rowptr, ci[order].to(torch.int32), w[order]

    def load(self, a: torch.Tensor, b: torch.Tensor, w: Optional[torch.Tensor] = None):
        """exchange + index_mapping + to_csr.  Returns (rowptr, col, val, rm, cm)."""
        if w is None:
            w = torch.ones(a.numel(), dtype=torch.float32, device=a.device)
        a2, b2, w2 = self.exchange(a, b, w)
        ri, ci, rm, cm = self.index_mapping(a2, b2)
        rowptr, col, val = self.to_csr(ri, ci, w2, rm.numel())
        return rowptr, col, val, rm, cm
