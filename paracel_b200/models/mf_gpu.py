"""Biased matrix factorisation by SGD on GPUs with the parameter-server shards
in HBM (device path of the reference's ``matrix_factorization`` paralg class,
alg/recommendation/matrix_factorization/mf.hpp:46-378).

One training round keeps the reference's structure (mf.hpp:282-323):

    read_mf_paras   -> RowTable.pull   (peer loads; SSP staleness wait fused in)
    local SGD pass  -> pcl_mf_sgd_pass (user-major chunks, vector reductions)
    update_mf_fac / update_mf_bias
                    -> RowTable.push   (wgt * (new - old) reduced into the owner)
    iter_commit     -> DeviceSspClock.commit

``wgt`` is 1 / (number of ranks that hold the row), gathered through a counter
table exactly like the reference's ``<id>_u_cnt`` / ``<id>_i_cnt`` keys
(mf.hpp:150-197).  Ratings are placed on a ``npx x npy`` rank grid by
(user group, item group) (the reference's ``fsmap`` pattern,
include/load/scheduler.hpp:81-92); groups can be balanced by rating mass so
that heavy-tailed id distributions do not overload one rank.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..parallel.ssp_device import DeviceSspClock
from ..ps.tables import RowTable, ScalarTable
from ..utils.decomp import npfact2d


def _pad_rank(k: int) -> int:
    for d in (32, 64, 128, 256):
        if k <= d:
            return d
    raise ValueError("factor rank above 256 is not supported by the SGD kernel")


def balanced_groups(counts: torch.Tensor, ngroups: int, spread_above: float = 0.0) -> torch.Tensor:
    """Assign ids to ``ngroups`` groups with near-equal total count.

    The ``heavy`` ids (count above 1/(64*ngroups) of the total) are placed greedily, largest
    first, on the lightest group.  The light tail then fills every group up to the common
    target: a tail id goes to group g with a share proportional to the group's remaining
    deficit, spread evenly over the popularity ranks by a golden-ratio sequence (so a group
    that already holds a very popular id receives few tail ids instead of an equal part).

    ``spread_above`` > 0 marks ids whose count exceeds ``spread_above / ngroups`` of the total
    with group -1: their entries are meant to be dealt over ALL groups by the other coordinate
    (see :func:`grid_rank`), which keeps one extremely popular row from making one group of
    ranks spend most of its pass on a single row; their mass counts as evenly divided here.

    Returns an int32 group id per id.  With ``ngroups == 1`` everything is group 0.
    """
    n = counts.numel()
    dev = counts.device
    grp = (torch.arange(n, device=dev, dtype=torch.int64) % ngroups).to(torch.int32)
    if ngroups == 1:
        return grp
    total = float(counts.sum().item())
    c64 = counts.to(torch.float64)
    spread = torch.zeros(n, dtype=torch.bool, device=dev)
    if spread_above > 0.0:
        spread = c64 > (spread_above / ngroups) * total
    spread_mass = float(c64[spread].sum().item())
    thresh = total / (64.0 * ngroups)
    heavy = torch.nonzero((c64 > thresh) & ~spread).flatten()
    load = torch.full((ngroups,), spread_mass / ngroups, dtype=torch.float64)
    g_heavy = torch.empty(heavy.numel(), dtype=torch.int32)
    if heavy.numel():
        hc = c64[heavy]
        order = torch.argsort(hc, descending=True)
        heavy, hc = heavy[order].cpu(), hc[order].cpu()
        for j in range(heavy.numel()):
            g = int(torch.argmin(load))
            g_heavy[j] = g
            load[g] += hc[j]
    light_mask = ~spread
    if heavy.numel():
        light_mask[heavy.to(dev)] = False
    light = torch.nonzero(light_mask).flatten()
    deficit = torch.clamp(total / ngroups - load, min=0.0)
    if float(deficit.sum()) <= 0.0:
        deficit = torch.ones(ngroups, dtype=torch.float64)
    edges = (torch.cumsum(deficit, 0) / deficit.sum()).to(dev)
    edges[-1] = 1.0
    x = torch.frac(torch.arange(light.numel(), device=dev, dtype=torch.float64) * 0.6180339887498949)
    grp[light] = torch.clamp(torch.searchsorted(edges, x, right=True), max=ngroups - 1).to(torch.int32)
    if heavy.numel():
        grp[heavy.to(dev)] = g_heavy.to(dev)
    grp[spread] = -1
    return grp


def grid_rank(u: torch.Tensor, i: torch.Tensor, ugrp: torch.Tensor, igrp: torch.Tensor,
              npx: int, npy: int) -> torch.Tensor:
    """Rank (grid row * npy + grid column) of every rating under the group tables of
    :func:`balanced_groups`.  The ratings of a user (item) marked -1 are dealt round-robin over
    the grid rows (columns) by their position in the list, so that row is shared by every rank
    of the grid row (column) whatever the popularity of the other coordinate."""
    gu = ugrp[u].to(torch.int64)
    gi = igrp[i].to(torch.int64)
    pos = torch.arange(u.numel(), device=u.device, dtype=torch.int64)
    gu = torch.where(gu < 0, pos % npx, gu)
    gi = torch.where(gi < 0, (pos // npx) % npy, gi)   # independent of the row dealt above
    return gu * npy + gi


class MfSgdGpu:
    def __init__(self, n_users: int, n_items: int, k: int = 128, alpha: float = 0.005,
                 beta: float = 0.02, rounds: int = 1, staleness: int = 2, ssp: bool = True,
                 group=None, device=None, seed: int = 0, hot_mix: float = 1.0,
                 sgd_blocks: int = 0, timeout_s: float = 5.0, hot_rows: int = 106,
                 chunks_per_flush: int = 8, variant: int = 0, compact: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        self.n_users, self.n_items, self.k = int(n_users), int(n_items), int(k)
        self.D = _pad_rank(self.k)
        self.alpha, self.beta = float(alpha), float(beta)
        self.rounds = int(rounds)
        self.staleness = int(staleness) if ssp else 0
        self.ssp = bool(ssp)
        self.seed = seed
        self.hot_mix = float(hot_mix)
        # variant 0: automatic (rank 128 -> sixteen-lanes-per-rating kernel, else the 32-lane one);
        # variant 1: 32-lanes-per-rating kernel, 2 CTAs per SM with 16 chunks in flight each;
        # variant 2 (D = 128): experimental 8-lanes-per-rating kernel, 1 CTA per SM, 64 chunks
        self.variant = int(variant)
        self.compact = bool(compact)
        self.g8 = (self.D == 128 and self.variant == 2)
        # variant 3 (D = 128): sixteen lanes per rating, two chunks per warp, 1 CTA of 640 threads per SM
        self.h16 = (self.D == 128 and self.variant in (0, 3))
        one_cta = self.g8 or self.h16
        self.sgd_blocks = int(sgd_blocks) if sgd_blocks > 0 else (148 if one_cta else 148 * 2)
        self.h16_threads = int(os.environ.get("PCL_MF_H16_THREADS", "640"))
        self.warps_per_block = 64 if self.g8 else (self.h16_threads // 16 if self.h16 else 16)   # chunks in flight per CTA
        self.hot_rows = int(hot_rows)
        self.chunks_per_flush = int(chunks_per_flush)
        self.npx, self.npy = npfact2d(self.world)
        self.px, self.py = self.rank // self.npy, self.rank % self.npy
        # parameter-server tables (shards in HBM)
        self.Wt = RowTable(self.n_users, self.D, torch.float32, group, self.device)
        self.Ht = RowTable(self.n_items, self.D, torch.float32, group, self.device)
        self.but = ScalarTable(self.n_users, group, self.device)
        self.bit = ScalarTable(self.n_items, group, self.device)
        self.clock = DeviceSspClock(self.staleness, self.rounds, group, self.device, timeout_s)
        self.mu = 0.0
        self.nnz = 0
        self.sse = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.host_stream = None
        self.h2d_bytes = 0
        self._loaded = False
        # optional (PCL_MF_OVERLAP_PUSH=1): push + commit of round t on a side stream, overlapped with
        # the SGD pass of round t+1; off by default since the push itself takes well under a millisecond
        self.overlap_push = os.environ.get("PCL_MF_OVERLAP_PUSH", "0") == "1"
        self._push_stream = None
        self._push_done = None
        # optional per-phase device timing of round() (diagnostics; adds event records only)
        self.phase_timing = False
        self._phase_events = []

    # ------------------------------------------------------------------ data
    def owner_of(self, ugrp: torch.Tensor, igrp: torch.Tensor) -> torch.Tensor:
        return ugrp.to(torch.int64) * self.npy + igrp.to(torch.int64)

    def load_ratings(self, u: torch.Tensor, i: torch.Tensor, r: torch.Tensor,
                     keep_on_host: bool = False):
        """Take this rank's ratings (global ids) and build the device layout.

        The ratings are sorted user-major, padded to whole chunks of 32 and the
        chunks are shuffled once, so that the chunks of one heavy user are
        spread over the pass and ratings are still read sequentially.  With
        ``keep_on_host`` the chunked arrays are kept in pinned host memory and
        streamed to the GPU every round (out-of-core mode).
        """
        dev = self.device
        u = u.to(dev, torch.int64)
        i = i.to(dev, torch.int64)
        r = r.to(dev, torch.float32)
        nnz = u.numel()
        self.nnz = nnz
        self.lu, ru = torch.unique(u, return_inverse=True)
        self.li, ri = torch.unique(i, return_inverse=True)
        cu = torch.bincount(ru, minlength=self.lu.numel())
        ci = torch.bincount(ri, minlength=self.li.numel())
        # resident warps = expected number of ratings in flight at any time
        P = self.sgd_blocks * self.warps_per_block
        # hot items: those that several resident warps would update at once; they
        # take the first local indices and are replicated in shared memory
        conc = P * ci.to(torch.float64) / max(nnz, 1)
        T = int(min(self.hot_rows, int((conc > 1.0).sum().item()), self.li.numel()))
        if self.g8:
            T = min(T, (220 * 1024) // ((2 * 132 + 2) * 4))
        elif self.h16:
            T = min(T, (220 * 1024) // ((2 * 128 + 2) * 4))
        else:
            T = min(T, (110 * 1024) // ((2 * self.D + 2) * 4))
        self.hot_T = T
        if T > 0:
            hot = torch.topk(ci, T).indices
            mask = torch.ones(ci.numel(), dtype=torch.bool, device=dev)
            mask[hot] = False
            new_order = torch.cat([hot, torch.nonzero(mask).flatten()])
            inv = torch.empty_like(new_order)
            inv[new_order] = torch.arange(new_order.numel(), device=dev)
            ri = inv[ri]
            self.li = self.li[new_order]
            ci = ci[new_order]
        self.li_sorted, self.li_perm = torch.sort(self.li)
        order = torch.argsort(ru, stable=True)
        ru, ri, r = ru[order].to(torch.int32), ri[order].to(torch.int32), r[order]
        del order
        pad = (-nnz) % 32
        if pad:
            ru = torch.cat([ru, torch.full((pad,), -1, dtype=torch.int32, device=dev)])
            ri = torch.cat([ri, torch.zeros(pad, dtype=torch.int32, device=dev)])
            r = torch.cat([r, torch.zeros(pad, dtype=torch.float32, device=dev)])
        nch = ru.numel() // 32
        g = torch.Generator(device=dev)
        g.manual_seed(self.seed * 7919 + 17 + self.rank)
        perm = torch.randperm(nch, device=dev, generator=g)
        ru = ru.view(nch, 32)[perm].contiguous().view(-1)
        ri = ri.view(nch, 32)[perm].contiguous().view(-1)
        r = r.view(nch, 32)[perm].contiguous().view(-1)
        del perm
        self.nchunks = nch
        self._build_compact(ru, ri, r)
        # concurrency weights (see csrc/cuda/mf.cu): expected number of resident
        # warps that touch the same row at the same time
        P = min(P, max(nch, 1))
        denom = max(nnz, 1)
        self.su = (1.0 / torch.clamp(self.hot_mix * P * cu.to(torch.float32) / denom, min=1.0)).contiguous()
        conc_i = torch.full((ci.numel(),), float(P), device=dev)
        conc_i[: self.hot_T] = float(min(self.warps_per_block, P))  # replicas: per-CTA concurrency
        self.si = (1.0 / torch.clamp(self.hot_mix * conc_i * ci.to(torch.float32) / denom, min=1.0)).contiguous()
        nU, nI = self.lu.numel(), self.li.numel()
        # user rows are shared by the ranks of this grid row, item rows by those of this grid
        # column: every sharer starts its push at a different place of the (sorted) id list
        stagger = os.environ.get("PCL_MF_STAGGER", "1") != "0"
        self._start_u = (self.py * nU) // max(self.npy, 1) if stagger else 0
        self._start_i = (self.px * nI) // max(self.npx, 1) if stagger else 0
        self.Wl = torch.empty(nU, self.D, device=dev)
        self.W0 = torch.empty(nU, self.D, device=dev)
        self.Hl = torch.empty(nI, self.D, device=dev)
        self.H0 = torch.empty(nI, self.D, device=dev)
        self.bul = torch.empty(nU, device=dev)
        self.bu0 = torch.empty(nU, device=dev)
        self.bil = torch.empty(nI, device=dev)
        self.bi0 = torch.empty(nI, device=dev)
        if keep_on_host:
            self.h_ru = ru.cpu().pin_memory()
            self.h_ri = ri.cpu().pin_memory()
            self.h_rr = r.cpu().pin_memory()
            self.ru = self.ri = self.rr = None
            if self.packed is not None:
                self.h_packed = self.packed.cpu().pin_memory()
                self.h_chdr = self.chdr.cpu().pin_memory()
                self.packed = self.chdr = None
        else:
            self.ru, self.ri, self.rr = ru, ri, r
            self.h_ru = None
        self._sum_r = float(r.sum(dtype=torch.float64).item())
        self._loaded = True

    def _build_compact(self, ru, ri, r):
        """Compact rating stream (4 bytes per rating + 12 per chunk): item index and an 8-bit
        rating code in one word; the users of a chunk as first index + increment mask (the users
        of a user-major sorted chunk grow by 0 or 1 per rating).  Used when there are at most
        2^24 local items and 256 distinct rating values."""
        self.packed = self.chdr = self.rtable = None
        self.h_packed = self.h_chdr = None
        if ru.numel() == 0:
            return
        vals = torch.unique(r)
        if self.li.numel() > (1 << 24) or vals.numel() > 256:
            return

        def as_i32(x):  # keep the low 32 bits of an int64 tensor as an int32 bit pattern
            return torch.where(x >= (1 << 31), x - (1 << 32), x).to(torch.int32)
        nch = ru.numel() // 32
        code = torch.searchsorted(vals, r).to(torch.int64)
        self.packed = as_i32((code << 24) | ri.to(torch.int64)).contiguous()
        u2 = ru.view(nch, 32).to(torch.int64)
        valid = u2 >= 0
        n_valid = valid.sum(1)
        first = torch.where(n_valid > 0, u2[:, 0], torch.full_like(n_valid, -1))
        prev = torch.cat([u2[:, :1], u2[:, :-1]], dim=1)
        inc = ((u2 - prev) == 1) & valid
        weights = (1 << torch.arange(32, device=ru.device, dtype=torch.int64))
        mask = as_i32((inc.to(torch.int64) * weights[None, :]).sum(1))
        self.chdr = torch.stack([first.to(torch.int32), mask, n_valid.to(torch.int32)], dim=1).contiguous().view(-1)
        self.rtable = torch.zeros(256, device=ru.device)
        self.rtable[: vals.numel()] = vals

    def offload_ratings(self):
        """Switch to out-of-core mode: move the chunked ratings to pinned host memory."""
        if self.h_ru is not None:
            return
        torch.cuda.synchronize(self.device)
        self.h_ru = self.ru.cpu().pin_memory()
        self.h_ri = self.ri.cpu().pin_memory()
        self.h_rr = self.rr.cpu().pin_memory()
        self.ru = self.ri = self.rr = None
        if self.packed is not None:
            self.h_packed = self.packed.cpu().pin_memory()
            self.h_chdr = self.chdr.cpu().pin_memory()
            self.packed = self.chdr = None

    # ------------------------------------------------------------ parameters
    def init_parameters(self):
        """Owner-side initialisation: factors U(0, 0.1), biases 0.1*U(0,1), mu = global
        mean rating (mf.hpp:127-143), then the holder counts -> push weights."""
        assert self._loaded
        dev = self.device
        g = torch.Generator(device=dev)
        g.manual_seed(self.seed * 1000003 + self.rank)
        for t, rows in ((self.Wt, self.n_users), (self.Ht, self.n_items)):
            t.shard.zero_()
            t.shard[:, : self.k] = 0.1 * torch.rand(t.rows_per_shard, self.k, device=dev, generator=g)
        self.but.shard.copy_(0.1 * torch.rand(self.but.rows_per_shard, device=dev, generator=g))
        self.bit.shard.copy_(0.1 * torch.rand(self.bit.rows_per_shard, device=dev, generator=g))
        tot = torch.tensor([self._sum_r, float(self.nnz)], dtype=torch.float64, device=dev)
        if self.world > 1:
            dist.all_reduce(tot, group=self.group)
        self.mu = float(tot[0].item() / max(tot[1].item(), 1.0))
        self.total_nnz = int(tot[1].item())
        # holder counts through counter tables
        cu = ScalarTable(self.n_users, self.group, dev)
        ci = ScalarTable(self.n_items, self.group, dev)
        ones_u = torch.ones(self.lu.numel(), device=dev)
        ones_i = torch.ones(self.li.numel(), device=dev)
        cu.push(self.lu, ones_u)
        ci.push(self.li, ones_i)
        self._barrier()
        cnt_u = torch.empty_like(ones_u)
        cnt_i = torch.empty_like(ones_i)
        cu.pull(self.lu, cnt_u)
        ci.pull(self.li, cnt_i)
        self.wgt_u = (1.0 / cnt_u.clamp(min=1.0)).contiguous()
        self.wgt_i = (1.0 / cnt_i.clamp(min=1.0)).contiguous()
        self._barrier()
        cu.free()
        ci.free()
        self._have_cache = False

    def _barrier(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    # ----------------------------------------------------------------- round
    def pull(self, fused_wait: bool = True):
        target = self.clock.wait_target() if (self.world > 1 and fused_wait) else 0
        self.Wt.pull(self.lu, self.Wl, self.W0, self.clock.clocks, target,
                     self.clock.timeout_ns, self.clock.status)
        self.Ht.pull(self.li, self.Hl, self.H0)
        self.but.pull(self.lu, self.bul, self.bu0)
        self.bit.pull(self.li, self.bil, self.bi0)
        self._have_cache = True

    def sgd_pass(self):
        s = _lib.stream_ptr()
        if self.h_ru is None and self.h16:
            pk = self.packed if self.compact else None
            _lib.call("pcl_mf_sgd_pass_h16", self.ru, self.ri, self.rr, self.ru.numel(), self.Wl, self.Hl,
                      self.bul, self.bil, self.su, self.si, self.mu, self.alpha, self.beta, self.hot_T,
                      self.chunks_per_flush, 0.0, self.sgd_blocks, self.sse, pk,
                      self.chdr if pk is not None else None, self.rtable if pk is not None else None,
                      self.h16_threads, s)
        elif self.h_ru is None:
            pk = self.packed if (self.compact and not self.g8) else None
            _lib.call("pcl_mf_sgd_pass", self.ru, self.ri, self.rr, self.ru.numel(), self.Wl,
                      self.Hl, self.bul, self.bil, self.su, self.si, self.D, self.mu,
                      self.alpha, self.beta, self.hot_T, self.chunks_per_flush, 0.0,
                      self.sgd_blocks, self.sse, self.variant, pk, self.chdr if pk is not None else None,
                      self.rtable if pk is not None else None, s)
        else:
            self._sgd_pass_streamed()

    def _sgd_pass_streamed(self, nseg: int = 16):
        """Out-of-core pass: ratings come from pinned host memory in segments; the copy of
        segment s+1 overlaps the SGD kernel of segment s (two staging buffers).  With the compact
        stream a segment is one int32 per rating plus three per chunk, otherwise three arrays."""
        dev = self.device
        n = self.h_ru.numel()
        compact = self.compact and not self.g8 and self.h_packed is not None
        seg = ((n // 32 + nseg - 1) // nseg) * 32
        if self.host_stream is None:
            self.host_stream = torch.cuda.Stream(device=dev)
            if compact:
                self._stage = [(torch.empty(seg, dtype=torch.int32, device=dev),
                                torch.empty(3 * (seg // 32), dtype=torch.int32, device=dev)) for _ in range(2)]
            else:
                self._stage = [(torch.empty(seg, dtype=torch.int32, device=dev),
                                torch.empty(seg, dtype=torch.int32, device=dev),
                                torch.empty(seg, dtype=torch.float32, device=dev)) for _ in range(2)]
            self._copied = [torch.cuda.Event() for _ in range(2)]
            self._consumed = [torch.cuda.Event() for _ in range(2)]
        main = torch.cuda.current_stream(dev)
        self.h2d_bytes = 0
        k = 0
        for off in range(0, n, seg):
            m = min(seg, n - off)
            b = k % 2
            with torch.cuda.stream(self.host_stream):
                if k >= 2:
                    self.host_stream.wait_event(self._consumed[b])
                if compact:
                    bpk, bhd = self._stage[b]
                    bpk[:m].copy_(self.h_packed[off:off + m], non_blocking=True)
                    c0, c1 = 3 * (off // 32), 3 * ((off + m) // 32)
                    bhd[: c1 - c0].copy_(self.h_chdr[c0:c1], non_blocking=True)
                    self.h2d_bytes += 4 * m + 4 * (c1 - c0)
                else:
                    bru, bri, brr = self._stage[b]
                    bru[:m].copy_(self.h_ru[off:off + m], non_blocking=True)
                    bri[:m].copy_(self.h_ri[off:off + m], non_blocking=True)
                    brr[:m].copy_(self.h_rr[off:off + m], non_blocking=True)
                    self.h2d_bytes += 12 * m
                self._copied[b].record(self.host_stream)
            main.wait_event(self._copied[b])
            if compact:
                seg_args = (None, None, None, bpk, bhd, self.rtable)
            else:
                seg_args = (bru, bri, brr, None, None, None)
            if self.h16:
                _lib.call("pcl_mf_sgd_pass_h16", seg_args[0], seg_args[1], seg_args[2], m, self.Wl, self.Hl,
                          self.bul, self.bil, self.su, self.si, self.mu, self.alpha, self.beta, self.hot_T,
                          self.chunks_per_flush, 0.0, self.sgd_blocks, self.sse, seg_args[3], seg_args[4],
                          seg_args[5], self.h16_threads, main.cuda_stream)
            else:
                _lib.call("pcl_mf_sgd_pass", seg_args[0], seg_args[1], seg_args[2], m, self.Wl, self.Hl,
                          self.bul, self.bil, self.su, self.si, self.D, self.mu, self.alpha, self.beta,
                          self.hot_T, self.chunks_per_flush, 0.0, self.sgd_blocks, self.sse, self.variant,
                          seg_args[3], seg_args[4], seg_args[5], main.cuda_stream)
            self._consumed[b].record(main)
            k += 1

    def push(self):
        self.Wt.push(self.lu, self.Wl, self.W0, self.wgt_u)
        self.Ht.push(self.li, self.Hl, self.H0, self.wgt_i)
        self.but.push(self.lu, self.bul, self.bu0, self.wgt_u)
        self.bit.push(self.li, self.bil, self.bi0, self.wgt_i)

    def need_pull(self) -> bool:
        """SSP cache rule (include/ps.hpp:437-457): first and last read always pull; with
        staleness s a cached copy may be reused while it is less than s clocks old."""
        c = self.clock.clock
        if not self._have_cache or not self.ssp or self.staleness == 0:
            return True
        if c == 0 or c >= self.rounds:
            return True
        return (c - self._pulled_at) >= self.staleness

    def _mark(self, label: str):
        if self.phase_timing:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._phase_events.append((label, e))

    def _push_sync(self):
        self.Wt.push(self.lu, self.Wl, self.W0, self.wgt_u, start=self._start_u)
        self._mark("push_W")
        self.Ht.push(self.li, self.Hl, self.H0, self.wgt_i, start=self._start_i)
        self._mark("push_H")
        self.but.push(self.lu, self.bul, self.bu0, self.wgt_u)
        self.bit.push(self.li, self.bil, self.bi0, self.wgt_i)
        self._mark("push_bias")
        if not self.ssp and self.world > 1:
            self._barrier()
        self.clock.commit()
        self._mark("commit")

    def _push_overlapped(self):
        """Push + commit on a side stream while the main stream goes on with the next round.

        The working copies are first copied to staging buffers (local, one pass); the side
        stream then reduces ``wgt * (staged - snapshot)`` into the owners' shards, refreshes
        the snapshots and commits the clock.  The peers' reductions arrive while every GPU is
        busy with its next SGD pass instead of holding the round up.  Used with a staleness
        bound of at least 2: this rank's own clock may then lag one commit behind without
        ever blocking its own wait."""
        dev = self.device
        main = torch.cuda.current_stream(dev)
        if self._push_stream is None:
            self._push_stream = torch.cuda.Stream(device=dev)
            self._Ws = torch.empty_like(self.Wl)
            self._Hs = torch.empty_like(self.Hl)
            self._bus = torch.empty_like(self.bul)
            self._bis = torch.empty_like(self.bil)
        if self._push_done is not None:
            main.wait_event(self._push_done)      # staging buffers are free again
        self._Ws.copy_(self.Wl)
        self._Hs.copy_(self.Hl)
        self._bus.copy_(self.bul)
        self._bis.copy_(self.bil)
        staged = torch.cuda.Event()
        staged.record(main)
        self._mark("stage")
        with torch.cuda.stream(self._push_stream):
            self._push_stream.wait_event(staged)
            self.Wt.push(self.lu, self._Ws, self.W0, self.wgt_u, start=self._start_u)
            self.Ht.push(self.li, self._Hs, self.H0, self.wgt_i, start=self._start_i)
            self.but.push(self.lu, self._bus, self.bu0, self.wgt_u)
            self.bit.push(self.li, self._bis, self.bi0, self.wgt_i)
            self.clock.commit()
            self._push_done = torch.cuda.Event()
            self._push_done.record(self._push_stream)

    def round(self):
        self._mark("start")
        if self.need_pull():
            if self._push_done is not None:       # the pull must see this rank's own pushes
                torch.cuda.current_stream(self.device).wait_event(self._push_done)
            self.pull()
            self._pulled_at = self.clock.clock
        elif self.world > 1:
            self.clock.wait()  # keep the staleness bound while serving from the cache
        self._mark("pull_or_wait")
        self.sse.zero_()
        self.sgd_pass()
        self._mark("sgd")
        if self.overlap_push and self.world > 1 and self.ssp and self.staleness >= 2:
            self._push_overlapped()
        else:
            self._push_sync()

    def phase_times_ms(self):
        """Mean device time of each phase of round() over the rounds run since ``phase_timing``
        was switched on (synchronises)."""
        torch.cuda.synchronize(self.device)
        out: Dict[str, float] = {}
        rounds = 0
        prev = None
        for label, e in self._phase_events:
            if label == "start":
                rounds += 1
            else:
                out[label] = out.get(label, 0.0) + prev.elapsed_time(e)
            prev = e
        out = {k: v / max(rounds, 1) for k, v in out.items()}
        out["rounds"] = rounds
        self._phase_events = []
        return out

    def fit(self):
        for _ in range(self.rounds):
            self.round()
        self._barrier()
        self.clock.check()
        self.pull(fused_wait=False)
        self._barrier()

    # --------------------------------------------------------------- metrics
    def running_rmse(self) -> float:
        """RMSE of the pre-update errors seen by the last SGD pass (8-byte D2H read)."""
        tot = self.sse.clone()
        if self.world > 1:
            dist.all_reduce(tot, group=self.group)
        return math.sqrt(float(tot.item()) / max(self.total_nnz, 1))

    def rmse(self) -> float:
        """Training RMSE of the clipped estimate with the current working copies
        (cal_rmse, mf.hpp:94-108)."""
        out = torch.zeros(1, dtype=torch.float64, device=self.device)
        ru, ri, rr = self._device_ratings()
        _lib.call("pcl_mf_sse", ru, ri, rr, ru.numel(), self.Wl, self.Hl, self.bul, self.bil,
                  self.D, self.mu, out, None, _lib.stream_ptr())
        # padding entries have u < 0 and predict mu against rating 0: remove them
        pad = ru.numel() - self.nnz
        out -= pad * (self.mu ** 2)
        if self.world > 1:
            dist.all_reduce(out, group=self.group)
        return math.sqrt(max(float(out.item()), 0.0) / max(self.total_nnz, 1))

    def _device_ratings(self):
        if self.h_ru is None:
            return self.ru, self.ri, self.rr
        dev = self.device
        return self.h_ru.to(dev), self.h_ri.to(dev), self.h_rr.to(dev)

    def predict(self, u: torch.Tensor, i: torch.Tensor) -> torch.Tensor:
        """Clipped estimate for (user, item) pairs by global id; unseen ids predict mu."""
        dev = self.device
        u = u.to(dev, torch.int64)
        i = i.to(dev, torch.int64)
        pu = torch.searchsorted(self.lu, u).clamp(max=max(self.lu.numel() - 1, 0))
        pi = torch.searchsorted(self.li_sorted, i).clamp(max=max(self.li.numel() - 1, 0))
        ok = (self.lu[pu] == u) & (self.li_sorted[pi] == i)
        pi = self.li_perm[pi]
        pu = torch.where(ok, pu, torch.full_like(pu, -1)).to(torch.int32).contiguous()
        pi = torch.where(ok, pi, torch.full_like(pi, -1)).to(torch.int32).contiguous()
        pred = torch.empty(u.numel(), device=dev)
        _lib.call("pcl_mf_sse", pu, pi, None, u.numel(), self.Wl, self.Hl, self.bul, self.bil,
                  self.D, self.mu, None, pred, _lib.stream_ptr())
        return pred

    # ------------------------------------------------------------------ dump
    def dump_result(self, outdir: str, user_names=None, item_names=None):
        """Write miu_0, ubias_0, ibias_0, W_0, H_0 in the reference's text layout
        (mf.hpp:380-492): rank 0 writes what each owner holds, shard by shard.  ``user_names`` /
        ``item_names`` (arrays indexed by the dense id) give the ids to print."""
        from ..utils.dump import dump_dict_scalar, dump_dict_vector
        os.makedirs(outdir, exist_ok=True)
        self._barrier()
        parts = {}
        for name, t, width in (("W_", self.Wt, self.k), ("H_", self.Ht, self.k)):
            ids = t.owned_ids().cpu()
            vals = t.shard[: ids.numel(), :width].cpu()
            parts[name] = (ids, vals)
        for name, t in (("ubias_", self.but), ("ibias_", self.bit)):
            ids = t.owned_ids().cpu()
            parts[name] = (ids, t.shard[: ids.numel()].cpu())
        gathered = [parts]
        if self.world > 1:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, parts, group=self.group)
        if self.rank == 0:
            dump_dict_scalar({"miu": self.mu, "rating_sz": float(self.total_nnz)},
                             os.path.join(outdir, "miu_0"))
            def keys(name, ids):
                tab = user_names if name in ("ubias_", "W_") else item_names
                return ids.tolist() if tab is None else [int(tab[j]) for j in ids.tolist()]
            for name in ("ubias_", "ibias_"):
                with open(os.path.join(outdir, name + "0"), "w") as f:
                    for p in gathered:
                        ids, vals = p[name]
                        dump_dict_scalar(dict(zip(keys(name, ids), vals.tolist())), f)
            for name in ("W_", "H_"):
                with open(os.path.join(outdir, name + "0"), "w") as f:
                    for p in gathered:
                        ids, vals = p[name]
                        dump_dict_vector(dict(zip(keys(name, ids), vals.tolist())), f)
        self._barrier()

    def free(self):
        self._barrier()
        for t in (self.Wt, self.Ht, self.but, self.bit, self.clock):
            t.free()
