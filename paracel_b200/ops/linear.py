"""Gradient kernels of the linear models (``csrc/cuda/linear.cu``)."""
from __future__ import annotations


import torch

from . import _lib


class DenseGrad:
    """g = X^T (y - h(X theta)) and the summed loss for dense fp32 X (row-major)."""

    def __init__(self, d: int, device, blocks: int = 592):
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
                  delta_l1=None, old_rank=None, threads_per_row: int = 8, heavy_rows=None,
                  heavy_deg: int = 2048):
    """``heavy_rows`` (int32 list of rows with more than ``heavy_deg`` in-links) are reduced by a
    whole thread block each instead of ``threads_per_row`` threads."""
    n = row_ptr.numel() - 1
    nh = 0 if heavy_rows is None else heavy_rows.numel()
    _lib.call("pcl_pagerank_pull", row_ptr, cols, contrib, inv_outdeg, n, float(damping), new_contrib,
              new_rank, delta_l1, old_rank, threads_per_row, int(heavy_deg), heavy_rows, nh,
              _lib.stream_ptr())


PR_CAPS = (2048, 4096)


def pagerank_stream_plan(row_ptr, cap: int = 2048):
    """Static per-graph plan of the edge-balanced kernel: for every block of ``cap`` in-links (2048
    or 4096) the row that holds its first and the row that holds its last in-link (int32 arrays),
    and ``cap`` itself."""
    if cap not in PR_CAPS:
        raise ValueError(f"cap must be one of {PR_CAPS}")
    nnz = int(row_ptr[-1].item())
    nb = (nnz + cap - 1) // cap
    if nb == 0:
        z = row_ptr.new_zeros(0, dtype=torch.int32)
        return z, z, cap
    starts = torch.arange(nb, device=row_ptr.device, dtype=torch.int64) * cap
    lasts = torch.clamp(starts + cap, max=nnz) - 1
    first = torch.searchsorted(row_ptr, starts, right=True) - 1
    last = torch.searchsorted(row_ptr, lasts, right=True) - 1
    return first.to(torch.int32).contiguous(), last.to(torch.int32).contiguous(), cap


def pagerank_pull_stream(row_ptr, cols, contrib, inv_outdeg, damping, acc, new_contrib, new_rank=None,
                         delta_l1=None, old_rank=None, plan=None):
    """Edge-balanced pull step: blocks own equal numbers of in-links (good for power-law graphs).
    ``acc`` is a scratch vector with one float per local vertex; ``plan`` comes from
    :func:`pagerank_stream_plan` (computed on the fly when missing)."""
    n = row_ptr.numel() - 1
    if plan is None:
        plan = pagerank_stream_plan(row_ptr)
    _lib.call("pcl_pagerank_pull_stream", row_ptr, cols, contrib, inv_outdeg, n, cols.numel(),
              plan[0], plan[1], float(damping), acc, new_contrib, new_rank, delta_l1, old_rank,
              int(plan[2]), _lib.stream_ptr())
