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

Every kernel that takes ids checks them against the table's extent; an id
outside ``[0, rows)`` is skipped and reported through the table's status block,
which ``check()`` turns into :class:`~paracel_b200.ops._lib.BadDeviceId`.  A
push whose status block already holds an error (a staleness wait of the same
round that ran out) does nothing, so a rank that could not pull does not mix
stale copies into the shared tables.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import _lib
from ..parallel.symm import SymmBuffer

HANDLERS = {"add": 0, "scaled_add": 1, "max": 2, "assign": 3}


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
        self.status = _lib.new_status(self.device)

    def check(self, what: str = "row table"):
        """Synchronise and raise if a kernel on this table reported a bad id or a timed-out wait."""
        _lib.check_status(self.status, what)

    # global ids owned by this rank, in local-row order
    def owned_ids(self) -> torch.Tensor:
        ids = torch.arange(self.rows_per_shard, device=self.device, dtype=torch.int64)
        ids = ids * self.world + self.rank
        return ids[ids < self.rows]

    def pull(self, ids: torch.Tensor, out: torch.Tensor, snapshot: Optional[torch.Tensor] = None,
             clocks: Optional[torch.Tensor] = None, target: int = 0,
             timeout_ns: int = 2_000_000_000, status: Optional[torch.Tensor] = None):
        """``status``: block that the fused staleness wait and the id check report through
        (default: the table's own)."""
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.check_cuda(out, self.dtype, "out")
        n = ids.numel()
        assert out.numel() == n * self.width
        s = _lib.stream_ptr()
        st = self.status if status is None else status
        if self.dtype == torch.float32:
            _lib.call("pcl_rows_pull_f32", ids, self.buf.ptr_table, self.world, self.width, n,
                      out, snapshot, clocks, int(target), int(timeout_ns), st, self.rank,
                      self.rows, s)
        elif self.dtype == torch.int32:
            _lib.call("pcl_rows_pull_i32", ids, self.buf.ptr_table, self.world, self.width, n,
                      out, snapshot, self.rows, st, self.rank, s)
        else:
            raise TypeError(self.dtype)

    def push(self, ids: torch.Tensor, cur: torch.Tensor, old: Optional[torch.Tensor] = None,
             wgt: Optional[torch.Tensor] = None, handler: str = "add", scale: float = 1.0,
             refresh_old: bool = True, start: int = 0, status: Optional[torch.Tensor] = None):
        """``start``: first row of ``ids`` to visit (the kernel wraps around).  Ranks that push the
        same rows at the same time should pass different values.  Handler ``max`` needs values
        that are not NaN; ``assign`` stores ``cur`` (``paracel_write_multi``)."""
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.check_cuda(cur, self.dtype, "cur")
        n = ids.numel()
        assert cur.numel() == n * self.width
        s = _lib.stream_ptr()
        st = self.status if status is None else status
        if self.dtype == torch.float32:
            _lib.call("pcl_rows_push_f32", ids, self.buf.ptr_table, self.world, self.width, n,
                      cur, old, wgt, float(scale), HANDLERS[handler], int(refresh_old), int(start),
                      self.rows, st, self.rank, s)
        else:
            if handler != "add" or wgt is not None:
                raise ValueError("int32 tables support the add handler only")
            _lib.call("pcl_rows_push_i32", ids, self.buf.ptr_table, self.world, self.width, n,
                      cur, old, int(refresh_old), self.rows, st, self.rank, s)

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
        self.width, self.dtype = 1, torch.float32
        self.status = _lib.new_status(self.device)

    def check(self, what: str = "scalar table"):
        _lib.check_status(self.status, what)

    def owned_ids(self) -> torch.Tensor:
        ids = torch.arange(self.rows_per_shard, device=self.device, dtype=torch.int64)
        ids = ids * self.world + self.rank
        return ids[ids < self.rows]

    def pull(self, ids, out, snapshot=None, status=None):
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.call("pcl_scalars_pull_f32", ids, self.buf.ptr_table, self.world, ids.numel(),
                  out, snapshot, self.rows, self.status if status is None else status, self.rank,
                  _lib.stream_ptr())

    def push(self, ids, cur, old=None, wgt=None, refresh_old=True, handler: str = "add",
             status=None, **_ignored):
        _lib.check_cuda(ids, torch.int64, "ids")
        _lib.call("pcl_scalars_push_f32", ids, self.buf.ptr_table, self.world, ids.numel(),
                  cur, old, wgt, int(refresh_old), HANDLERS[handler], self.rows,
                  self.status if status is None else status, self.rank, _lib.stream_ptr())

    def free(self):
        self.shard = None
        self.buf.free()


DENSE_KINDS = {"add": 0, "sgd": 1, "prox_l1": 2, "max": 3}


def _dense_kind(name: str):
    """(kernel code, registered lr, registered lambda) of a handler name on a dense table."""
    from .device_handlers import resolve_device_handler
    h = resolve_device_handler(name)
    if h.kind == "scaled_add":          # theta += scale * sum  ==  sgd with lr = -scale
        return DENSE_KINDS["sgd"], -(h.scale if h.scale is not None else 1.0), h.lam
    if h.kind not in DENSE_KINDS:
        raise ValueError(f"handler {name!r} ({h.kind}) cannot run as a dense bupdate")
    return DENSE_KINDS[h.kind], h.lr, h.lam


class DenseTable:
    """One dense fp32 parameter vector of length ``L`` ("theta", cluster centres, a rank
    vector), range-sharded over the ranks: rank r owns elements ``[r*S, (r+1)*S)``.

    ``read()`` is ``paracel_read`` of the key: an all-gather into a local full copy by peer
    loads.  ``delta()`` is the local full-length buffer a gradient kernel writes into, and
    ``bupdate()`` is ``paracel_bupdate`` with the table's registered handler: every owner
    reduces its slice of all ranks' delta buffers out of peer memory and applies the handler
    in the same kernel (reduce-scatter fused with the update).  Ordering between ranks is
    carried by two flag arrays in peer memory ("delta ready", "update done") that the kernels
    wait on with a deadline; no host barrier is involved.
    """

    def __init__(self, L: int, group=None, device=None, handler: str = "add", lr: float = 1.0,
                 lam: float = 0.0, timeout_s: float = 5.0):
        import torch.distributed as dist
        self.L = int(L)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        S = (self.L + self.world - 1) // self.world
        self.S = (S + 3) // 4 * 4
        self.Lp = self.S * self.world
        self.theta_buf = SymmBuffer(self.S, torch.float32, group, device)
        self.delta_buf = SymmBuffer(2 * self.Lp, torch.float32, group, device)
        self.flag_buf = SymmBuffer(128, torch.int64, group, device)
        self.device = self.theta_buf.device
        self.shard = self.theta_buf.local
        self.full = torch.zeros(self.Lp, device=self.device)
        self.handler, self.lr, self.lam = handler, float(lr), float(lam)
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        self.status = torch.zeros(4, dtype=torch.int64, device=self.device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.nnz = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.count_nnz = False     # bupdate also counts the non-zeros of the new shard into nnz
        base = self.delta_buf.ptr_table
        self._delta_tables = [base.clone(), (base + self.Lp * 4).contiguous()]
        self._ready_table = self.flag_buf.ptr_table.clone()
        self._done_table = (self.flag_buf.ptr_table + 64 * 8).contiguous()
        self.ready = self.flag_buf.local[:64]
        self.done = self.flag_buf.local[64:]

    def owned_range(self):
        lo = self.rank * self.S
        return lo, min(self.L, lo + self.S)

    def delta(self) -> torch.Tensor:
        """Buffer (length L) for the delta of the NEXT bupdate."""
        b = (self.epoch + 1) & 1
        return self.delta_buf.local[b * self.Lp: b * self.Lp + self.L]

    def read(self, copy: bool = True) -> torch.Tensor:
        """The whole vector.  ``copy=False`` lets a single-rank table return a view of its
        shard (no kernel); callers that use it must not update the table while they hold it."""
        if not copy and self.world == 1:
            return self.shard[: self.L]
        _lib.call("pcl_dense_read", self.theta_buf.ptr_table, self.full, self.Lp, self.S, self.world,
                  self.rank, self.done, self.epoch, self.timeout_ns, self.status, _lib.stream_ptr())
        return self.full[: self.L]

    def bupdate(self, handler: Optional[str] = None, lr: Optional[float] = None,
                lam: Optional[float] = None, count_nnz: Optional[bool] = None):
        if count_nnz is None:
            count_nnz = self.count_nnz
        self.epoch += 1
        b = self.epoch & 1
        s = _lib.stream_ptr()
        _lib.call("pcl_publish_flag", self._ready_table, self.world, self.rank, self.epoch, s)
        h, reg_lr, reg_lam = _dense_kind(handler or self.handler)
        if lr is None:
            lr = self.lr if reg_lr is None else reg_lr
        if lam is None:
            lam = self.lam if reg_lam is None else reg_lam
        if count_nnz:
            self.nnz.zero_()
        _lib.call("pcl_dense_bupdate", self.shard, self._delta_tables[b], self.Lp, self.S, self.world,
                  self.rank, h, float(lr), float(lam), self.ready, self.epoch, self.timeout_ns,
                  self.status, self._done_table, self.counter, self.nnz if count_nnz else None, s)

    def mark_written(self):
        """The owner has rewritten its shard in place (e.g. a kernel stored new values there):
        publish that as the next epoch so that readers wait for every owner."""
        self.epoch += 1
        _lib.call("pcl_publish_flag", self._done_table, self.world, self.rank, self.epoch,
                  _lib.stream_ptr())

    def write(self, values: torch.Tensor):
        """Collective initialisation from a full vector that every rank passes identically: each
        owner stores its slice and publishes that as the next epoch, so the next ``read`` on any
        rank waits (bounded) until every owner has written."""
        lo, hi = self.owned_range()
        self.shard.zero_()
        if hi > lo:
            self.shard[: hi - lo] = values[lo:hi].to(self.device, torch.float32)
        self.mark_written()

    def push(self, delta: torch.Tensor, scale: float = 1.0):
        """One-sided update: this rank alone adds ``scale * delta`` (full length ``L``) into the
        owners' shards by reductions over NVLink.  Nothing waits; other ranks see the result
        after the next synchronisation (``paracel_sync`` or a clock commit)."""
        _lib.check_cuda(delta, torch.float32, "delta")
        if delta.numel() != self.L:
            raise ValueError(f"delta has {delta.numel()} elements, the table {self.L}")
        _lib.call("pcl_dense_push", self.theta_buf.ptr_table, delta, self.L, self.S, self.world,
                  self.rank, float(scale), _lib.stream_ptr())

    def check(self):
        _lib.check_status(self.status, "dense table")

    def free(self):
        self.shard = None
        self.ready = self.done = None
        for b in (self.theta_buf, self.delta_buf, self.flag_buf):
            b.free()
