"""SSP clock kept in GPU memory (device replacement of the reference's SSP
server thread, include/server.hpp:114-167, and of the client-side polling in
include/ps.hpp:343-355, 447-457).

Every rank owns ``clocks[world]`` (int64) in a symmetric buffer.  ``commit``
stores the rank's new clock into slot ``rank`` of every peer's array with one
tiny kernel; ``wait`` (or the wait fused into ``RowTable.pull``) spins, with a
deadline, until ``min(clocks) >= clock - staleness``.  When the deadline passes
the kernel records what it saw in a status block and returns; the host turns
that into :class:`SspTimeout`.  Nothing here can hang a GPU.
"""
from __future__ import annotations

import torch

from ..ops import _lib
from .symm import SymmBuffer

DEPARTED = (1 << 62)


class SspTimeout(RuntimeError):
    def __init__(self, rank, wait_id, expected, seen):
        super().__init__(f"rank {rank}: SSP wait {wait_id} timed out: need min clock >= "
                         f"{expected}, saw {seen}")
        self.rank, self.wait_id, self.expected, self.seen = rank, wait_id, expected, seen


class DeviceSspClock:
    def __init__(self, staleness: int, total_iters: int, group=None, device=None,
                 timeout_s: float = 2.0):
        self.buf = SymmBuffer(64, torch.int64, group, device)  # world <= 64 ranks per box
        self.world, self.rank = self.buf.world, self.buf.rank
        if self.world > 64:
            raise ValueError("DeviceSspClock supports at most 64 ranks")
        self.clocks = self.buf.local
        self.staleness = int(staleness)
        self.total_iters = int(total_iters)
        self.clock = 0
        self.timeout_ns = int(timeout_s * 1e9)
        # status block: PclStatus = 4 ints + 2 long longs = 32 bytes
        self.status = torch.zeros(4, dtype=torch.int64, device=self.buf.device)

    def wait_target(self) -> int:
        """Smallest min-clock that lets this rank start iteration ``self.clock``."""
        return max(0, self.clock - self.staleness)

    def commit(self):
        self.clock += 1
        value = DEPARTED if self.clock >= self.total_iters else self.clock
        _lib.call("pcl_ssp_commit", self.buf.ptr_table, self.world, self.rank, value, self.status,
                  _lib.stream_ptr())

    def restore(self, clock: int):
        """Resume at ``clock`` (collective, after a checkpoint load): set the local counter and
        store the value into every peer's clock array, as the commit that ended iteration
        ``clock - 1`` did."""
        self.clock = int(clock)
        value = DEPARTED if self.clock >= self.total_iters else self.clock
        _lib.call("pcl_ssp_commit", self.buf.ptr_table, self.world, self.rank, value, self.status,
                  _lib.stream_ptr())

    def wait(self):
        _lib.call("pcl_ssp_wait", self.clocks, self.world, self.wait_target(), self.timeout_ns,
                  self.status, self.rank, _lib.stream_ptr())

    def check(self):
        """Synchronise and raise what the status block holds since the last check: SspTimeout for
        a wait that expired, BadDeviceId when a pull or push that reported through this block met
        an id outside its table."""
        st = self.status.cpu()
        code = int(st[0].item()) & 0xFFFFFFFF
        if code == 0:
            return
        lo = int(st[0].item())
        rank = (lo >> 32) & 0xFFFFFFFF
        wait_id = int(st[1].item()) & 0xFFFFFFFF
        expected, seen = int(st[2].item()), int(st[3].item())
        self.status.zero_()
        if code == 2:
            raise _lib.BadDeviceId("device table", rank, wait_id, expected, seen)
        raise SspTimeout(rank, wait_id, expected, seen)

    def free(self):
        self.clocks = None
        self.buf.free()
