"""fp32-storage GEMM on the tcgen05 tensor cores (``csrc/cuda/gemm_tf32.cu``).

``gemm_nt(A, B)`` returns ``A @ B.T`` for row-major fp32 ``A [M, K]`` and
``B [N, K]``.  ``precise=True`` evaluates the error-compensated 3xTF32 form
(three tf32 products per element, fp32-level accuracy) by splitting both
operands into tf32-exact high and low parts along K.  ``argmin_nt`` fuses the
row-wise ``argmin_n (bnorm[n] - 2 A.B^T)`` of k-means into the epilogue.

``DenseReadGemm`` is the multi-rank form: B is a parameter that is
range-sharded over the ranks (rank r owns rows ``[r*rps, (r+1)*rps)``); the
kernel gathers the peers' shards over NVLink into a local staging buffer while
the tensor cores already work on the tiles that have arrived.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ..parallel.symm import SymmBuffer


# "2sm": pairs of CTAs on one 256 x 256 (or 256 x 512) item (tcgen05 cta_group::2,
#        gemm_tf32_2sm.cu);
# "1sm": one CTA per 128 x 128 tile (gemm_tf32.cu).
KERNEL = os.environ.get("PCL_GEMM_KERNEL", "2sm")
# item form of the pair kernel: 1 = 256 x 512 (two accumulators share an A stage), 0 = 256 x 256
# with alternating accumulators, -1 = the launcher chooses by K
WIDE = int(os.environ.get("PCL_GEMM_WIDE", "-1"))


def _entry(kernel: Optional[str] = None) -> str:
    k = kernel or KERNEL
    if k not in ("1sm", "2sm"):
        raise ValueError(f"unknown GEMM kernel {k!r}")
    return "pcl_gemm_tf32_2sm" if k == "2sm" else "pcl_gemm_tf32"


def _pad_k(x: torch.Tensor) -> torch.Tensor:
    k = x.shape[1]
    if k % 4 == 0 and x.is_contiguous() and x.data_ptr() % 16 == 0:
        return x
    kp = (k + 3) // 4 * 4
    out = torch.zeros(x.shape[0], kp, device=x.device, dtype=torch.float32)
    out[:, :k] = x
    return out


def split3(x: torch.Tensor, is_b: bool) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty(x.shape[0], 3 * x.shape[1], device=x.device, dtype=torch.float32)
    _lib.call("pcl_split3_tf32", x, out, x.shape[0], x.shape[1], int(is_b), _lib.stream_ptr())
    return out


_STATUS = {}


def _status(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    st = _STATUS.get(key)
    if st is None:
        st = _STATUS[key] = torch.zeros(4, dtype=torch.int64, device=device)
    return st


def check_status(device=None) -> None:
    """Raise if a GEMM launched by ``gemm_nt`` / ``argmin_nt`` on ``device`` gave up on a wait
    (synchronises the device)."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    st = _STATUS.get(dev.index or 0)
    if st is None:
        return
    host = st.cpu()
    if int(host[0].item()) & 0xFFFFFFFF:
        st.zero_()
        raise RuntimeError(f"GEMM wait timed out: wait id {int(host[1].item()) & 0xFFFFFFFF}, "
                           f"expected {int(host[2])}, saw {int(host[3])}")


def _merge_halves(rm2: torch.Tensor, ra2: torch.Tensor):
    """The two-CTA kernel reports the arg-min per half of the columns of a tile; keep the smaller
    (the lower column index on ties)."""
    m0, m1, a0, a1 = rm2[0], rm2[1], ra2[0], ra2[1]
    take1 = (m1 < m0) | ((m1 == m0) & (a1 < a0))
    return torch.where(take1, m1, m0), torch.where(take1, a1, a0)


def _launch(A, B, C, epi, bnorm, row_min, row_arg, status=None, kernel=None, wide=None):
    M, K = A.shape
    if status is None:
        status = _status(A.device)
    N = B.shape[0]
    ldc = C.stride(0) if C is not None else 0
    entry = _entry(kernel)
    if entry == "pcl_gemm_tf32_2sm":
        _lib.call(entry, A, B, C, M, N, K, ldc, epi, bnorm, row_min, row_arg, None, None, 1, 0,
                  N, 0, 0, status, 0, WIDE if wide is None else int(wide), _lib.stream_ptr())
        return
    _lib.call(entry, A, B, C, M, N, K, ldc, epi, bnorm, row_min, row_arg, None, None, 1, 0,
              N, 0, 0, status, 0, _lib.stream_ptr())


def gemm_nt(A: torch.Tensor, B: torch.Tensor, out: Optional[torch.Tensor] = None,
            precise: bool = False, kernel: Optional[str] = None,
            wide: Optional[int] = None) -> torch.Tensor:
    _lib.check_cuda(A, torch.float32, "A")
    _lib.check_cuda(B, torch.float32, "B")
    assert A.shape[1] == B.shape[1]
    M, N = A.shape[0], B.shape[0]
    if precise:
        A2, B2 = split3(_pad_k(A), False), split3(_pad_k(B), True)
    else:
        A2, B2 = _pad_k(A), _pad_k(B)
    if out is None:
        out = torch.empty(M, N, device=A.device, dtype=torch.float32)
    _launch(A2, B2, out, 0, None, None, None, kernel=kernel, wide=wide)
    return out


def argmin_nt(A: torch.Tensor, B: torch.Tensor, bnorm: Optional[torch.Tensor] = None,
              precise: bool = False, kernel: Optional[str] = None,
              wide: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(min value of bnorm[n] - 2 a.b_n, its index n) per row of A."""
    _lib.check_cuda(A, torch.float32, "A")
    _lib.check_cuda(B, torch.float32, "B")
    if bnorm is None:
        bnorm = (B * B).sum(1)
    bnorm = bnorm.contiguous()
    M = A.shape[0]
    if precise:
        A2, B2 = split3(_pad_k(A), False), split3(_pad_k(B), True)
    else:
        A2, B2 = _pad_k(A), _pad_k(B)
    two = _entry(kernel) == "pcl_gemm_tf32_2sm"
    row_min = torch.empty((2, M) if two else (M,), device=A.device, dtype=torch.float32)
    row_arg = torch.empty((2, M) if two else (M,), device=A.device, dtype=torch.int32)
    _launch(A2, B2, None, 1, bnorm, row_min, row_arg, kernel=kernel, wide=wide)
    return _merge_halves(row_min, row_arg) if two else (row_min, row_arg)


class DenseReadGemm:
    """All-gather of a range-sharded B [N, K] fused with A @ B.T.

    ``shard`` (this rank's rows of B) lives in a symmetric buffer; ``__call__`` may be
    invoked repeatedly (every call re-reads the peers' current shards).  The caller must
    make sure nobody writes the shards while a call is in flight (barrier or SSP clock).
    """

    def __init__(self, N: int, K: int, group=None, device=None, gather_ctas: int = 8,
                 kernel: Optional[str] = None, wide: Optional[int] = None):
        if K % 4:
            raise ValueError("K must be a multiple of 4")
        self.N, self.K = N, K
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rps = (N + self.world - 1) // self.world
        self.buf = SymmBuffer(self.rps * K, torch.float32, group, device)
        self.shard = self.buf.local.view(self.rps, K)
        self.device = self.buf.device
        self.stage = torch.zeros(N, K, device=self.device)
        self.flags = torch.zeros((N + 127) // 128, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int64, device=self.device)
        self.epoch = 0
        self.gather_ctas = gather_ctas
        self.entry = _entry(kernel)
        self.wide = WIDE if wide is None else int(wide)

    @property
    def _tail(self):
        # trailing launcher arguments: the pair kernel takes its tile form before the stream
        if self.entry == "pcl_gemm_tf32_2sm":
            return (self.wide, _lib.stream_ptr())
        return (_lib.stream_ptr(),)

    def local_rows(self) -> Tuple[int, int]:
        lo = self.rank * self.rps
        return lo, min(self.N, lo + self.rps)

    def __call__(self, A: torch.Tensor, out: Optional[torch.Tensor] = None,
                 argmin_bnorm: Optional[torch.Tensor] = None):
        _lib.check_cuda(A, torch.float32, "A")
        assert A.shape[1] == self.K
        M = A.shape[0]
        self.epoch += 1
        if self.world == 1:
            stage, shards = self.shard, None
        else:
            stage, shards = self.stage, self.buf.ptr_table
        if argmin_bnorm is None:
            if out is None:
                out = torch.empty(M, self.N, device=A.device, dtype=torch.float32)
            _lib.call(self.entry, A, stage, out, M, self.N, self.K, out.stride(0), 0, None, None,
                      None, shards, self.flags, self.world, self.rank, self.rps, self.epoch,
                      self.gather_ctas, self.status, 0, *self._tail)
            return out
        two = self.entry == "pcl_gemm_tf32_2sm"
        row_min = torch.empty((2, M) if two else (M,), device=A.device, dtype=torch.float32)
        row_arg = torch.empty((2, M) if two else (M,), device=A.device, dtype=torch.int32)
        _lib.call(self.entry, A, stage, None, M, self.N, self.K, 0, 1, argmin_bnorm, row_min,
                  row_arg, shards, self.flags, self.world, self.rank, self.rps, self.epoch,
                  self.gather_ctas, self.status, 0, *self._tail)
        return _merge_halves(row_min, row_arg) if two else (row_min, row_arg)

    def check(self):
        st = self.status.cpu()
        if int(st[0].item()) & 0xFFFFFFFF:
            self.status.zero_()
            raise RuntimeError(f"fused gather+GEMM wait timed out: wait id "
                               f"{int(st[1].item()) & 0xFFFFFFFF}, expected {int(st[2])}, saw {int(st[3])}")

    def free(self):
        self.shard = None
        self.buf.free()
