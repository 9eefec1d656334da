"""Gradient kernels of the linear models (``csrc/cuda/linear.cu``)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


class DenseGrad:
    """g = X^T (y - h(X theta)) and the summed loss for dense fp32 X (row-major)."""

    def __init__(self, d: int, device, blocks: int = 296):
        self.d, self.blocks = d, blocks
        self.scratch = torch.empty(blocks * d + 2 * blocks + 4, device=device, dtype=torch.float32)
        self.counter = torch.zeros(1, device=device, dtype=torch.int32)
        self.loss = torch.zeros(1, device=device, dtype=torch.float64)

    def __call__(self, X, y, theta, g, logistic: bool = True):
        _lib.check_cuda(X, torch.float32, "X")
        n, d = X.shape
        assert d == self.d and g.numel() >= d
        _lib.call("pcl_lr_dense_grad", X, y, theta, n, d, int(logistic), g, self.loss, self.scratch,
                  self.counter, self.blocks, _lib.stream_ptr())
        return self.loss


def sparse_grad(row_ptr, cols, vals, y, theta, g, loss, logistic: bool = True, hot_T: int = 8192,
                blocks: int = 0):
    """Accumulate g += X^T (y - h(X theta)) and loss for a CSR matrix (int64 row_ptr, int32 cols)."""
    n = row_ptr.numel() - 1
    hot_T = min(hot_T, g.numel())
    _lib.call("pcl_lr_sparse_grad", row_ptr, cols, vals, y, theta, n, int(logistic), hot_T, g, loss,
              blocks, _lib.stream_ptr())


def pagerank_pull(row_ptr, cols, contrib, inv_outdeg, damping, new_contrib, new_rank=None,
                  delta_l1=None, old_rank=None, threads_per_row: int = 8):
    n = row_ptr.numel() - 1
    _lib.call("pcl_pagerank_pull", row_ptr, cols, contrib, inv_outdeg, n, float(damping), new_contrib,
              new_rank, delta_l1, old_rank, threads_per_row, _lib.stream_ptr())
