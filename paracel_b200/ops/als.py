"""Batched ALS solve (``csrc/cuda/als.cu``): W[u] = (H_u^T H_u + lambda I)^-1 H_u^T a_u."""
from __future__ import annotations

import torch

from . import _lib


def _kpad(k: int) -> int:
    for K in (32, 64, 96, 128):
        if k <= K:
            return K
    raise ValueError("factor rank above 128 is not supported")


def als_solve(user_ptr: torch.Tensor, item_idx: torch.Tensor, rating: torch.Tensor, H: torch.Tensor,
              lam: float, seg_len: int = 4096) -> torch.Tensor:
    """``user_ptr`` (int64, n_users + 1) delimits each user's entries of ``item_idx`` (int32 rows
    of H) and ``rating`` (fp32).  Users with more than ``seg_len`` ratings are split over
    several CTAs.  Returns W [n_users, k]."""
    dev = H.device
    H = H.contiguous().float()
    n_users, k = user_ptr.numel() - 1, H.shape[1]
    # the kernel gathers rows of H by these indices without looking at them again
    _lib.validate_ids(item_idx.contiguous(), 0, H.shape[0], "ALS ratings (item rows)")
    K = _kpad(k)
    W = torch.zeros(n_users, k, device=dev)
    cnt = (user_ptr[1:] - user_ptr[:-1])
    nseg = torch.clamp((cnt + seg_len - 1) // seg_len, min=1)
    nseg = torch.where(cnt > 0, nseg, torch.zeros_like(nseg))
    total = int(nseg.sum().item())
    if total == 0:
        return W
    seg_user = torch.repeat_interleave(torch.arange(n_users, device=dev), nseg)
    first = torch.cumsum(nseg, 0) - nseg
    within = torch.arange(total, device=dev) - first[seg_user]
    seg_begin = user_ptr[:-1][seg_user] + within * seg_len
    seg_end = torch.minimum(seg_begin + seg_len, user_ptr[1:][seg_user])
    split = nseg > 1
    n_slots = int(split.sum().item())
    slot = torch.full((n_users,), -1, dtype=torch.int32, device=dev)
    slot[split] = torch.arange(n_slots, dtype=torch.int32, device=dev)
    scratch = torch.zeros(max(n_slots, 1) * (K * K + K), device=dev)
    counts = torch.zeros(max(n_slots, 1), dtype=torch.int32, device=dev)
    _lib.call("pcl_als_solve", seg_user.int().contiguous(), seg_begin.contiguous(), seg_end.contiguous(),
              nseg.int().contiguous(), slot, item_idx.int().contiguous(), rating.float().contiguous(), H, W,
              scratch, counts, total, k, float(lam), 0, _lib.stream_ptr())
    return W
