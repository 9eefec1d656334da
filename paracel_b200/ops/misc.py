"""Wrappers of the smaller kernels in ``csrc/cuda/misc.cu``."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ..parallel.symm import SymmBuffer


def kmeans_accumulate(X: torch.Tensor, assign: torch.Tensor, sums: torch.Tensor, counts: torch.Tensor):
    """sums[c] += X[i], counts[c] += 1 for c = assign[i]."""
    _lib.check_cuda(X, torch.float32, "X")
    _lib.check_cuda(assign, torch.int32, "assign")
    _lib.call("pcl_kmeans_accumulate", X, assign, X.shape[0], X.shape[1], sums, counts, _lib.stream_ptr())


class RunningTopK:
    """Per-row top-k (k <= 32) over a stream of similarity tiles, with a lower bound and
    exclusion of the row's own id."""

    def __init__(self, row_ids: torch.Tensor, k: int, lower: float = -3.0e38):
        self.row_ids = row_ids.to(torch.int64).contiguous()
        self.k, self.lower = int(k), float(lower)
        m = self.row_ids.numel()
        self.val = torch.full((m, k), -3.402823466e38, device=row_ids.device)
        self.idx = torch.full((m, k), -1, dtype=torch.int64, device=row_ids.device)

    def update(self, S: torch.Tensor, col_ids: torch.Tensor):
        _lib.check_cuda(S, torch.float32, "S")
        _lib.call("pcl_topk_rows", S, S.stride(0), S.shape[0], S.shape[1], self.row_ids,
                  col_ids.to(torch.int64).contiguous(), self.lower, self.k, self.val, self.idx,
                  _lib.stream_ptr())

    def result(self):
        """{row id: [(col id, value), ...]} best first, without empty slots."""
        out = {}
        v, i, r = self.val.cpu(), self.idx.cpu(), self.row_ids.cpu()
        for a in range(r.numel()):
            lst = [(int(i[a, j]), float(v[a, j])) for j in range(self.k) if int(i[a, j]) >= 0]
            if lst:
                out[int(r[a])] = lst
        return out


def gram(H: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """H^T H (k <= 128) accumulated into ``out`` (created zeroed when not given)."""
    _lib.check_cuda(H, torch.float32, "H")
    k = H.shape[1]
    if out is None:
        out = torch.zeros(k, k, device=H.device)
    _lib.call("pcl_gram", H, H.shape[0], k, out, _lib.stream_ptr())
    return out


class DeviceAllReduce:
    """Sum of a small fp64 vector over all ranks in one kernel launch: every rank stages its
    values in its own symmetric slot, publishes an epoch flag to its peers, waits (bounded) for
    theirs and adds up the peers' slots with peer loads."""

    def __init__(self, nmax: int = 256, group=None, device=None, timeout_s: float = 5.0):
        self.nmax = nmax
        self.slots = SymmBuffer(2 * nmax, torch.float64, group, device)
        self.flags = SymmBuffer(256, torch.int64, group, device)
        self.world, self.rank, self.device = self.slots.world, self.slots.rank, self.slots.device
        self.epoch = 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.status = torch.zeros(4, dtype=torch.int64, device=self.device)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _lib.check_cuda(x, torch.float64, "x")
        if out is None:
            out = torch.empty_like(x)
        self.epoch += 1
        _lib.call("pcl_allreduce_sum_f64", x, out, x.numel(), self.slots.ptr_table, self.flags.ptr_table,
                  self.flags.local, self.world, self.rank, self.nmax, self.epoch, self.timeout_ns,
                  self.status, _lib.stream_ptr())
        return out

    def check(self):
        st = self.status.cpu()
        if int(st[0].item()) & 0xFFFFFFFF:
            self.status.zero_()
            raise RuntimeError("device all-reduce timed out waiting for a peer")

    def free(self):
        self.slots.free()
        self.flags.free()
