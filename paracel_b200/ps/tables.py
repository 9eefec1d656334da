"""Typed parameter tables whose shards live in GPU memory.

``RowTable`` holds ``rows`` fixed-width rows (fp32 or int32).  Row ``g`` is
owned by rank ``g % world`` and stored at local row ``g // world`` of that
rank's :class:`~paracel_b200.parallel.symm.SymmBuffer`, so a key's placement is
arithmetic instead of the reference's consistent-hash ring lookup
(include/ring.hpp:85-92).  ``pull`` and ``push`` are the bulk forms of
``paracel_read_multi`` / ``paracel_bupdate_multi`` (include/ps.hpp:482-534,
810-871) executed by one kernel each over NVLink peer pointers; the handler
registered for the table (add, scaled add, max) runs at the owner as part of
the reduction.

``ScalarTable`` is the width-1 case (biases, counters).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import _lib
from ..parallel.symm import SymmBuffer

HANDLERS = {"add": 0, "scaled_add": 1, "max": 2}


class RowTable:
    def __init__(self, rows: int, width: int, dtype=torch.float32, group=None, device=None):
        if width % 4 != 0:
            raise ValueError("row width must be a multiple of 4 elements (16 bytes)")
        self.rows, self.width, self.dtype = int(rows), int(width), dtype
        import torch.distributed as dist
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows_per_shard = (self.rows + self.world - 1) // self.world
        self.buf = SymmBuffer(self.rows_per_shard * self.width, dtype, group, device)
        self.shard = self.buf.local.view(self.rows_per_shard, self.width)
        self.device = self.buf.device

    # global ids owned by this rank, in local-row order
    def owned_ids(self) -> torch.Tensor:
        ids = torch.arange(self.rows_per_shard, device=self.device, dtype=torch.int64)
        ids = ids * self.world + self.rank
        return ids[ids < self.rows]

    def pull(self, ids: torch.Tensor, out: torch.Tensor, snapshot: Optional[torch.Tensor] = None,
             clocks: Optional[torch.Tensor] = None, target: int = 0,
             timeout_ns: int = 2_000_000_000, status: Optional[torch.Tensor] = None):
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.check_cuda(out, self.dtype, "out")
        n = ids.numel()
        assert out.numel() == n * self.width
        s = _lib.stream_ptr()
        if self.dtype == torch.float32:
            _lib.call("pcl_rows_pull_f32", ids, self.buf.ptr_table, self.world, self.width, n,
                      out, snapshot, clocks, int(target), int(timeout_ns), status, self.rank, s)
        elif self.dtype == torch.int32:
            _lib.call("pcl_rows_pull_i32", ids, self.buf.ptr_table, self.world, self.width, n,
                      out, snapshot, s)
        else:
            raise TypeError(self.dtype)

    def push(self, ids: torch.Tensor, cur: torch.Tensor, old: Optional[torch.Tensor] = None,
             wgt: Optional[torch.Tensor] = None, handler: str = "add", scale: float = 1.0,
             refresh_old: bool = True):
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.check_cuda(cur, self.dtype, "cur")
        n = ids.numel()
        s = _lib.stream_ptr()
        if self.dtype == torch.float32:
            _lib.call("pcl_rows_push_f32", ids, self.buf.ptr_table, self.world, self.width, n,
                      cur, old, wgt, float(scale), HANDLERS[handler], int(refresh_old), s)
        else:
            if handler != "add" or wgt is not None:
                raise ValueError("int32 tables support the add handler only")
            _lib.call("pcl_rows_push_i32", ids, self.buf.ptr_table, self.world, self.width, n,
                      cur, old, int(refresh_old), s)

    def free(self):
        self.shard = None
        self.buf.free()


class ScalarTable:
    def __init__(self, rows: int, group=None, device=None):
        import torch.distributed as dist
        self.rows = int(rows)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows_per_shard = (self.rows + self.world - 1) // self.world
        self.buf = SymmBuffer(self.rows_per_shard, torch.float32, group, device)
        self.shard = self.buf.local
        self.device = self.buf.device

    def owned_ids(self) -> torch.Tensor:
        ids = torch.arange(self.rows_per_shard, device=self.device, dtype=torch.int64)
        ids = ids * self.world + self.rank
        return ids[ids < self.rows]

    def pull(self, ids, out, snapshot=None):
        _lib.call("pcl_scalars_pull_f32", ids, self.buf.ptr_table, self.world, ids.numel(),
                  out, snapshot, _lib.stream_ptr())

    def push(self, ids, cur, old=None, wgt=None, refresh_old=True):
        _lib.call("pcl_scalars_push_f32", ids, self.buf.ptr_table, self.world, ids.numel(),
                  cur, old, wgt, int(refresh_old), _lib.stream_ptr())

    def free(self):
        self.shard = None
        self.buf.free()
