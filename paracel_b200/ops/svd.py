"""Wrappers of the device SVD kernels (``csrc/cuda/svd.cu``): CSR x dense products with a
skinny right-hand side and the Cholesky factor of a small Gram matrix."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def spmm_csr(row_ptr: torch.Tensor, cols: torch.Tensor, vals: Optional[torch.Tensor], H: torch.Tensor,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``A @ H`` for CSR ``A`` (int64 row_ptr, int32 cols, fp32 vals or None for ones) and dense
    ``H [N, K]`` with ``K <= 128`` a multiple of 4."""
    _lib.check_cuda(H, torch.float32, "H")
    n, K = row_ptr.numel() - 1, H.shape[1]
    if out is None:
        out = torch.empty(n, K, device=H.device)
    _lib.call("pcl_spmm_csr", row_ptr, cols, vals, n, H, K, out, _lib.stream_ptr())
    return out


def spmm_csr_t(row_ptr: torch.Tensor, cols: torch.Tensor, vals: Optional[torch.Tensor], W: torch.Tensor,
               out: torch.Tensor) -> torch.Tensor:
    """``out += A.T @ W`` for CSR ``A`` with ``n`` rows and dense ``W [n, K]``; ``out [N, K]``."""
    _lib.check_cuda(W, torch.float32, "W")
    _lib.check_cuda(out, torch.float32, "out")
    n, K = row_ptr.numel() - 1, W.shape[1]
    _lib.call("pcl_spmm_csr_t", row_ptr, cols, vals, n, W, K, out, _lib.stream_ptr())
    return out


def chol_factor(G: torch.Tensor, rel_tol: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """For a symmetric positive definite ``G [K, K]`` (K <= 112): ``(T, R, info)`` with
    ``G = R^T R``, ``T = R^-1`` (so ``M T`` is orthonormal when ``G = M^T M`` and
    ``G^-1 = T T^T``).  ``info`` > 0 is the (1-based) pivot at which the factorisation met a
    value below ``rel_tol`` times the largest diagonal entry; T and R are then undefined."""
    _lib.check_cuda(G, torch.float32, "G")
    K = G.shape[0]
    T = torch.empty(K, K, device=G.device)
    R = torch.empty(K, K, device=G.device)
    info = torch.zeros(1, dtype=torch.int32, device=G.device)
    _lib.call("pcl_chol_factor", G, K, T, R, float(rel_tol), info, _lib.stream_ptr())
    return T, R, int(info.item())
