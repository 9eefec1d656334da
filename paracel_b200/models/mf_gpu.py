"""Biased matrix factorisation by SGD on GPUs with the parameter-server shards
in HBM (device path of the reference's ``matrix_factorization`` paralg class,
alg/recommendation/matrix_factorization/mf.hpp:46-378).

``MfSgdGpu`` is a ``paralg`` subclass on the device backend: the keys ``W_<uid>`` /
``H_<iid>`` / ``usr_bias_<uid>`` / ``item_bias_<iid>`` are rows of tables sharded over the
ranks' HBM, and one training round is the reference's round (mf.hpp:282-323) written with
the same calls:

    read_mf_paras   -> paracel_read_multi(keys, out=, snapshot=)   peer loads; the SSP
                                                                    staleness wait rides in the kernel
    local SGD pass  -> pcl_mf_sgd_pass (user-major chunks, vector reductions)
    update_mf_fac / update_mf_bias
                    -> paracel_bupdate_multi(keys, new, "", "mf_fac_updater", old=, wgt=)
                                                                    wgt * (new - old) reduced at the owner
    iter_commit     -> clock word stored into every peer's HBM

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
from ..paralg import paralg


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
              npx: int, npy: int, by_id: bool = False) -> torch.Tensor:
    """Rank (grid row * npy + grid column) of every rating under the group tables of
    :func:`balanced_groups`.  The ratings of a user (item) marked -1 are dealt over the grid
    rows (columns), so that row is shared by every rank of the grid row (column) whatever the
    popularity of the other coordinate: round-robin by their position in the list, or, with
    ``by_id``, by the id of the other coordinate (the same pair then always lands on the same
    rank, whoever computes it)."""
    gu = ugrp[u].to(torch.int64)
    gi = igrp[i].to(torch.int64)
    if by_id:
        gu = torch.where(gu < 0, i % npx, gu)
        gi = torch.where(gi < 0, (u // npx) % npy, gi)
        return gu * npy + gi
    pos = torch.arange(u.numel(), device=u.device, dtype=torch.int64)
    gu = torch.where(gu < 0, pos % npx, gu)
    gi = torch.where(gi < 0, (pos // npx) % npy, gi)   # independent of the row dealt above
    return gu * npy + gi


class RoundResult:
    """Result of one ``round()``: the squared pre-update error of its SGD pass.  The 8-byte copy
    to pinned host memory is queued right behind the pass, so ``sse()`` waits for that copy only
    and a caller that keeps one round in flight (queue round t + 1, then read round t) never lets
    the device run dry while the host reads.  The model keeps the results of its last four rounds;
    a handle that is older than that raises instead of returning another round's value."""
    __slots__ = ("_ev", "_host", "_model", "_no", "_val")

    def __init__(self, ev, host, model, no):
        self._ev, self._host, self._model, self._no, self._val = ev, host, model, no, None

    def sse(self) -> float:
        if self._val is None:
            if self._model._res_no - self._no >= self._model.RESULT_SLOTS:
                raise RuntimeError("this round's result slot has been reused: read a RoundResult "
                                   "within four rounds of the round that returned it")
            self._ev.synchronize()
            self._val = float(self._host.item())
        return self._val


class MfSgdGpu(paralg):
    RESULT_SLOTS = 4      # rounds whose RoundResult stays readable

    def __init__(self, n_users: int, n_items: int, k: int = 128, alpha: float = 0.005,
                 beta: float = 0.02, rounds: int = 1, staleness: int = 2, ssp: bool = True,
                 group=None, device=None, seed: int = 0, hot_mix: Optional[float] = None,
                 sgd_blocks: int = 0, timeout_s: float = 5.0, hot_rows: int = 106,
                 chunks_per_flush: int = 8, variant: int = 0, compact: bool = True,
                 comm=None, hosts_dct_str=None, output: str = "", user_names=None,
                 item_names=None, update_funcs=None, flush_scale: float = 0.0,
                 flush_mode: str = "uniform", grid=None, stream_segments: Optional[int] = None):
        super().__init__(hosts_dct_str, comm, output, int(rounds), int(staleness) if ssp else 0,
                         bool(ssp), wait_timeout_s=timeout_s, backend="gpu", device=device,
                         group=group)
        self.group = group
        self.world = self.get_worker_size()
        self.rank = self.get_worker_id()
        self.update_funcs = list(update_funcs or ["cnt_updater", "mf_fac_updater", "mf_bias_updater"])
        self.n_users, self.n_items, self.k = int(n_users), int(n_items), int(k)
        self.D = _pad_rank(self.k)
        self.alpha, self.beta = float(alpha), float(beta)
        self.rounds = int(rounds)
        self.staleness = int(staleness) if ssp else 0
        self.ssp = bool(ssp)
        self.seed = seed
        # The concurrency weights are 1 / max(1, hot_mix * expected concurrent updates of the row).
        # 1.0 damps a row by its full expected concurrency; 0.125 was the best of a sweep
        # (1, 0.5, 0.25, 0.125, 0.06, 0.03) of held-out RMSE per epoch on Zipf(1.1) ratings against
        # the sequential fp64 pass, and values below 0.06 start to oscillate.
        # (That sweep ran the 16-lanes-per-rating kernel; the other kernels keep 1.0 unless told.)
        self._hot_mix_arg = hot_mix
        # weight of a CTA's accumulated hot-row delta when it is mixed into the global row
        # (<= 0: 1 / number of CTAs, the plain average of the replicas)
        self.flush_scale = float(flush_scale)
        # "uniform": every hot row is mixed with flush_scale; "per_row": rows with fewer ratings
        # than the hottest take proportionally more of each CTA's delta (see load_ratings).
        # Measured on Zipf(1.1) ratings the per-row weights converge worse, so uniform is the default.
        self.flush_mode = flush_mode
        # variant 0: automatic (rank 128 -> sixteen-lanes-per-rating kernel, else the 32-lane one);
        # variant 1: 32-lanes-per-rating kernel, 2 CTAs per SM with 16 chunks in flight each;
        # variant 2 (D = 128): experimental 8-lanes-per-rating kernel, 1 CTA per SM, 64 chunks
        self.variant = int(variant)
        self.compact = bool(compact)
        self.allow_packed24 = os.environ.get("PCL_MF_PACKED24", "1") != "0"
        self.g8 = (self.D == 128 and self.variant == 2)
        # variant 3 (D = 128): sixteen lanes per rating, two chunks per warp, 1 CTA of 640 threads per SM
        self.h16 = (self.D == 128 and self.variant in (0, 3))
        self.hot_mix = float(self._hot_mix_arg) if self._hot_mix_arg is not None else (0.125 if self.h16 else 1.0)
        one_cta = self.g8 or self.h16
        self.sgd_blocks = int(sgd_blocks) if sgd_blocks > 0 else (148 if one_cta else 148 * 2)
        self.h16_threads = int(os.environ.get("PCL_MF_H16_THREADS", "640"))
        self.warps_per_block = 64 if self.g8 else (self.h16_threads // 16 if self.h16 else 16)   # chunks in flight per CTA
        self.hot_rows = int(hot_rows)
        self.chunks_per_flush = int(chunks_per_flush)
        # rank grid of the fsmap pattern: a user's ratings live on one grid row (npy ranks share
        # the user's row of W), an item's on one grid column (npx ranks share its row of H)
        # Default: the factorisation of the worker count that holds the fewest rows per rank,
        # n_users / npx + n_items / npy (every held row is pulled and pushed each round).  On
        # 8 GPUs with 1 M users x 200 k items that is 8 x 1: 47.4 G updates/s against 44.1 G for the
        # most square grid 2 x 4, and a lower held-out RMSE because W rows are no longer averaged
        # over four holders.
        if grid is None:
            grid = min(((a, self.world // a) for a in range(1, self.world + 1) if self.world % a == 0),
                       key=lambda g_: self.n_users / g_[0] + self.n_items / g_[1])
        self.npx, self.npy = int(grid[0]), int(grid[1])
        if self.npx * self.npy != self.world:
            raise ValueError(f"grid {self.npx} x {self.npy} does not match {self.world} workers")
        self.px, self.py = self.rank // self.npy, self.rank % self.npy
        # parameter tables (shards in HBM) behind the reference's key names
        self.user_names, self.item_names = user_names, item_names
        self.W_tab = self.paracel_row_table(self.n_users, self.D, prefix="W_", names=user_names,
                                            handler=self.update_funcs[1])
        self.H_tab = self.paracel_row_table(self.n_items, self.D, prefix="H_", names=item_names,
                                            handler=self.update_funcs[1])
        self.ub_tab = self.paracel_scalar_table(self.n_users, prefix="usr_bias_", names=user_names,
                                                handler=self.update_funcs[2])
        self.ib_tab = self.paracel_scalar_table(self.n_items, prefix="item_bias_", names=item_names,
                                                handler=self.update_funcs[2])
        # the tables themselves (owner-side initialisation, tests)
        self.Wt, self.Ht = self.W_tab.table, self.H_tab.table
        self.but, self.bit = self.ub_tab.table, self.ib_tab.table
        self.mu = 0.0
        self.nnz = 0
        # Segments per round when the ratings are streamed from host memory (offload_ratings);
        # None: as many as keep a staging buffer within 1 GiB, at least 2.  Every segment is a
        # kernel launch with its own replica set-up and tail (about 60 us): measured on 200 M
        # ratings (675 MB), 2 / 4 / 8 / 16 segments cost 0.1 / 0.25 / 0.5 / 1.4 ms on a 28.4 ms round.
        env_seg = os.environ.get("PCL_MF_STREAM_SEGMENTS")
        self.stream_segments = (int(stream_segments) if stream_segments is not None
                                else int(env_seg) if env_seg else None)
        self.sse = torch.zeros(1, dtype=torch.float64, device=self.device)
        # results of the last four rounds in pinned host memory (see RoundResult)
        self._sse_host = torch.zeros(self.RESULT_SLOTS, 1, dtype=torch.float64).pin_memory()
        self._sse_ev = [torch.cuda.Event() for _ in range(self.RESULT_SLOTS)]
        self._res_no = 0
        self.host_stream = None
        self.h2d_bytes = 0
        self._loaded = False
        # optional (PCL_MF_OVERLAP_PUSH=1): push + commit of round t on a side stream, overlapped with
        # the SGD pass of round t+1; off by default since the push itself takes well under a millisecond
        self.overlap_push = os.environ.get("PCL_MF_OVERLAP_PUSH", "0") == "1"
        self._push_stream = None
        self._push_done = None
        self.metrics_sync = False    # metrics lines also carry the pass's SSE (one D2H read per round)

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
            T = min(T, (220 * 1024) // ((144 + 128 + 2) * 4))   # delta rows are 144 words apart
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
        # Weight of one CTA's accumulated delta of a hot row when the replicas are mixed into the
        # global row.  The hottest row takes the plain average over the CTAs (1 / blocks); a
        # row with fewer ratings takes proportionally more, up to the full sum, so that every hot
        # row moves by about the same number of averaged steps per mixing period.
        self.hot_fs = None
        if self.h16 and self.hot_T > 0 and self.flush_mode == "per_row":
            nblk = min(self.sgd_blocks, max((nch + self.warps_per_block - 1) // self.warps_per_block, 1))
            top = float(ci[0].item())
            self.hot_fs = torch.clamp(top / ci[: self.hot_T].to(torch.float32).clamp(min=1.0) / nblk,
                                      max=1.0).contiguous()
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
            self._offload_compact()
        else:
            self.ru, self.ri, self.rr = ru, ri, r
            self.h_ru = None
        self._sum_r = float(r.sum(dtype=torch.float64).item())
        # the SGD kernel indexes the working copies with these local ids without looking at them
        # again: range-check them once, here
        if ru.numel():
            _lib.validate_ids(ru, 0, nU, "MF rating stream (user index)", skip=-1)
            _lib.validate_ids(ri, 0, nI, "MF rating stream (item index)")
        # key batches of this rank's rows
        self.kW = self.paracel_keys(self.W_tab, self.lu)
        self.kH = self.paracel_keys(self.H_tab, self.li)
        self.kub = self.paracel_keys(self.ub_tab, self.lu)
        self.kib = self.paracel_keys(self.ib_tab, self.li)
        self._loaded = True

    def _build_compact(self, ru, ri, r):
        """Compact rating stream: per rating the item index and a rating code in 3 bytes (21 + 3
        bits, when there are at most 2^21 local items and 8 distinct rating values) or in one
        word (24 + 8 bits, up to 2^24 items and 256 values); per chunk of 32 ratings 12 bytes for
        the users: first index + increment mask (the users of a user-major sorted chunk grow by
        0 or 1 per rating).  3.375 or 4.375 bytes per rating instead of 12."""
        self.packed = self.chdr = self.rtable = None
        self.h_packed = self.h_chdr = None
        # The one-word form feeds the kernel when the ratings are resident in HBM (its decode is
        # a mask and a shift); the three-byte form is what is streamed from host memory in
        # out-of-core mode, where the bytes of the copy set the pace.
        self.packed24 = None
        self.packed_bits = 32          # form of the stream that the host copy holds
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
        if self.h16 and self.allow_packed24 and self.li.numel() <= (1 << 21) and vals.numel() <= 8:
            # value e of a chunk occupies bits [24 e, 24 e + 24) of the chunk's 24 words
            v = (code << 21) | ri.to(torch.int64)
            b3 = torch.stack([v & 0xFF, (v >> 8) & 0xFF, (v >> 16) & 0xFF], dim=1).to(torch.uint8)
            self.packed24 = b3.view(nch, 96).contiguous().view(torch.int32).reshape(-1).contiguous()
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
        self._offload_compact()

    def _offload_compact(self):
        if self.packed is None:
            return
        src = self.packed24 if self.packed24 is not None else self.packed
        self.packed_bits = 24 if self.packed24 is not None else 32
        self.h_packed = src.cpu().pin_memory()
        self.h_chdr = self.chdr.cpu().pin_memory()
        self.packed = self.packed24 = self.chdr = None

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
        # holder counts through the keys <uid>_u_cnt / <iid>_i_cnt (mf.hpp:150-197)
        cu = self.paracel_scalar_table(self.n_users, suffix="_u_cnt", handler=self.update_funcs[0])
        ci = self.paracel_scalar_table(self.n_items, suffix="_i_cnt", handler=self.update_funcs[0])
        ku, ki = self.paracel_keys(cu, self.lu), self.paracel_keys(ci, self.li)
        self.paracel_bupdate_multi(ku, torch.ones(self.lu.numel(), device=dev), "", self.update_funcs[0])
        self.paracel_bupdate_multi(ki, torch.ones(self.li.numel(), device=dev), "", self.update_funcs[0])
        self.paracel_sync()
        cnt_u = self.paracel_read_multi(ku, ssp_wait=False)
        cnt_i = self.paracel_read_multi(ki, ssp_wait=False)
        self.wgt_u = (1.0 / cnt_u.clamp(min=1.0)).contiguous()
        self.wgt_i = (1.0 / cnt_i.clamp(min=1.0)).contiguous()
        self.paracel_sync()
        self.dev.drop(cu)
        self.dev.drop(ci)
        self.paracel_invalidate_cache()

    def _barrier(self):
        self.paracel_sync()

    # ----------------------------------------------------------------- round
    def read_mf_paras(self, ssp_wait: bool = True):
        """The local rows of W, H and the biases from their owners (mf.hpp:202-215), with a
        snapshot for the later delta push.  Under SSP the copies are reused while they are
        younger than the staleness bound."""
        self.paracel_read_multi(self.kW, out=self.Wl, snapshot=self.W0, ssp_wait=ssp_wait)
        self.paracel_read_multi(self.kH, out=self.Hl, snapshot=self.H0, ssp_wait=ssp_wait)
        self.paracel_read_multi(self.kub, out=self.bul, snapshot=self.bu0, ssp_wait=ssp_wait)
        self.paracel_read_multi(self.kib, out=self.bil, snapshot=self.bi0, ssp_wait=ssp_wait)

    def pull(self, fused_wait: bool = True):
        """Unconditional fresh read of the local rows (evaluation, the end of training)."""
        self.paracel_invalidate_cache()
        self.read_mf_paras(ssp_wait=fused_wait)

    def sgd_pass(self):
        s = _lib.stream_ptr()
        if self.h_ru is None and self.h16:
            pk = self.packed if self.compact else None
            _lib.call("pcl_mf_sgd_pass_h16", self.ru, self.ri, self.rr, self.ru.numel(), self.Wl, self.Hl,
                      self.bul, self.bil, self.su, self.si, self.mu, self.alpha, self.beta, self.hot_T,
                      self.chunks_per_flush, self.flush_scale, self.sgd_blocks, self.sse, pk,
                      self.chdr if pk is not None else None, self.rtable if pk is not None else None,
                      self.h16_threads, self.hot_fs, 32, s)
        elif self.h_ru is None:
            pk = self.packed if (self.compact and not self.g8) else None
            _lib.call("pcl_mf_sgd_pass", self.ru, self.ri, self.rr, self.ru.numel(), self.Wl,
                      self.Hl, self.bul, self.bil, self.su, self.si, self.D, self.mu,
                      self.alpha, self.beta, self.hot_T, self.chunks_per_flush, self.flush_scale,
                      self.sgd_blocks, self.sse, self.variant, pk, self.chdr if pk is not None else None,
                      self.rtable if pk is not None else None, s)
        else:
            nseg = self.stream_segments
            if nseg is None:
                # two staging buffers of at most 1 GiB each; never fewer than two segments, so that
                # the copy of one always runs under the kernel of the other
                compact = self.compact and not self.g8 and self.h_packed is not None
                stream_bytes = self.h_ru.numel() * (self.packed_bits / 8.0 if compact else 12.0)
                nseg = max(2, math.ceil(stream_bytes / float(1 << 30)))
            self._sgd_pass_streamed(nseg)

    def _sgd_pass_streamed(self, nseg: int):
        """Out-of-core pass: ratings come from pinned host memory in segments; the copy of
        segment s+1 overlaps the SGD kernel of segment s (two staging buffers), and the copy of
        the NEXT round's first segment is queued as soon as this round's last kernel is, so it
        runs under the push, the commit and the next pull instead of in front of the next pass.
        With the compact stream a segment is one int32 per rating plus three per chunk,
        otherwise three arrays.  Every round copies every rating once (``h2d_bytes``)."""
        dev = self.device
        n = self.h_ru.numel()
        compact = self.compact and not self.g8 and self.h_packed is not None
        seg = ((n // 32 + nseg - 1) // nseg) * 32
        if self.host_stream is None:
            self.host_stream = torch.cuda.Stream(device=dev)
            if compact:
                self._stage = [(torch.empty(seg * self.packed_bits // 32, dtype=torch.int32, device=dev),
                                torch.empty(3 * (seg // 32), dtype=torch.int32, device=dev)) for _ in range(2)]
            else:
                self._stage = [(torch.empty(seg, dtype=torch.int32, device=dev),
                                torch.empty(seg, dtype=torch.int32, device=dev),
                                torch.empty(seg, dtype=torch.float32, device=dev)) for _ in range(2)]
            self._copied = [torch.cuda.Event() for _ in range(2)]
            self._consumed = [None, None]       # recorded after the kernel that read the buffer
            self._seg_no = 0                    # running segment counter: buffer = counter % 2
            self._prefetched = False            # the first segment of this round is already on its way
        main = torch.cuda.current_stream(dev)

        def copy_segment(off, b):
            """Queue the copy of the segment at ``off`` into staging buffer ``b``; returns its bytes."""
            m = min(seg, n - off)
            with torch.cuda.stream(self.host_stream):
                if self._consumed[b] is not None:     # the kernel that last read this buffer is done
                    self.host_stream.wait_event(self._consumed[b])
                if compact:
                    bpk, bhd = self._stage[b]
                    w0, w1 = off * self.packed_bits // 32, (off + m) * self.packed_bits // 32
                    bpk[: w1 - w0].copy_(self.h_packed[w0:w1], non_blocking=True)
                    c0, c1 = 3 * (off // 32), 3 * ((off + m) // 32)
                    bhd[: c1 - c0].copy_(self.h_chdr[c0:c1], non_blocking=True)
                    nbytes = 4 * (w1 - w0) + 4 * (c1 - c0)
                else:
                    bru, bri, brr = self._stage[b]
                    bru[:m].copy_(self.h_ru[off:off + m], non_blocking=True)
                    bri[:m].copy_(self.h_ri[off:off + m], non_blocking=True)
                    brr[:m].copy_(self.h_rr[off:off + m], non_blocking=True)
                    nbytes = 12 * m
                self._copied[b].record(self.host_stream)
            return nbytes

        self.h2d_bytes = 0
        offs = list(range(0, n, seg))
        for j, off in enumerate(offs):
            m = min(seg, n - off)
            b = self._seg_no % 2
            if j == 0 and self._prefetched:
                self._prefetched = False
                self.h2d_bytes += self._prefetched_bytes
            else:
                self.h2d_bytes += copy_segment(off, b)
            main.wait_event(self._copied[b])
            if compact:
                bpk, bhd = self._stage[b]
                seg_args = (None, None, None, bpk, bhd, self.rtable)
            else:
                bru, bri, brr = self._stage[b]
                seg_args = (bru, bri, brr, None, None, None)
            if self.h16:
                _lib.call("pcl_mf_sgd_pass_h16", seg_args[0], seg_args[1], seg_args[2], m, self.Wl, self.Hl,
                          self.bul, self.bil, self.su, self.si, self.mu, self.alpha, self.beta, self.hot_T,
                          self.chunks_per_flush, self.flush_scale, self.sgd_blocks, self.sse, seg_args[3], seg_args[4],
                          seg_args[5], self.h16_threads, self.hot_fs, self.packed_bits, main.cuda_stream)
            else:
                _lib.call("pcl_mf_sgd_pass", seg_args[0], seg_args[1], seg_args[2], m, self.Wl, self.Hl,
                          self.bul, self.bil, self.su, self.si, self.D, self.mu, self.alpha, self.beta,
                          self.hot_T, self.chunks_per_flush, self.flush_scale, self.sgd_blocks, self.sse, self.variant,
                          seg_args[3], seg_args[4], seg_args[5], main.cuda_stream)
            ev = torch.cuda.Event()
            ev.record(main)
            self._consumed[b] = ev
            self._seg_no += 1
        if self.clock + 1 < self.rounds and offs:
            # next round's first segment: the bytes count towards that round
            self._prefetched_bytes = copy_segment(offs[0], self._seg_no % 2)
            self._prefetched = True

    def update_mf(self, start_u: int = 0, start_i: int = 0):
        """Push ``wgt * (new - old)`` of every local row to its owner (update_mf_fac /
        update_mf_bias, mf.hpp:217-262) and refresh the snapshots."""
        fac, bias = self.update_funcs[1], self.update_funcs[2]
        with self.phase("push_W"):
            self.paracel_bupdate_multi(self.kW, self.Wl, "", fac, old=self.W0, wgt=self.wgt_u, start=start_u)
        with self.phase("push_H"):
            self.paracel_bupdate_multi(self.kH, self.Hl, "", fac, old=self.H0, wgt=self.wgt_i, start=start_i)
        with self.phase("push_bias"):
            self.paracel_bupdate_multi(self.kub, self.bul, "", bias, old=self.bu0, wgt=self.wgt_u)
            self.paracel_bupdate_multi(self.kib, self.bil, "", bias, old=self.bi0, wgt=self.wgt_i)

    def push(self):
        self.update_mf()

    @property
    def phase_timing(self) -> bool:
        return self.timer is not None

    @phase_timing.setter
    def phase_timing(self, on: bool):
        """Per-phase device timing of round() (diagnostics; adds event records only)."""
        from ..utils.metrics import PhaseTimer
        self.timer = PhaseTimer() if on else None

    def _push_sync(self):
        self.update_mf(self._start_u, self._start_i)
        with self.phase("commit"):
            if not self.ssp and self.world > 1:
                self.paracel_sync()
            self.iter_commit()

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
        with self.phase("stage"):
            if self._push_done is not None:
                main.wait_event(self._push_done)      # staging buffers are free again
            self._Ws.copy_(self.Wl)
            self._Hs.copy_(self.Hl)
            self._bus.copy_(self.bul)
            self._bis.copy_(self.bil)
        staged = torch.cuda.Event()
        staged.record(main)
        fac, bias = self.update_funcs[1], self.update_funcs[2]
        with torch.cuda.stream(self._push_stream):
            self._push_stream.wait_event(staged)
            self.paracel_bupdate_multi(self.kW, self._Ws, "", fac, old=self.W0, wgt=self.wgt_u,
                                       start=self._start_u)
            self.paracel_bupdate_multi(self.kH, self._Hs, "", fac, old=self.H0, wgt=self.wgt_i,
                                       start=self._start_i)
            self.paracel_bupdate_multi(self.kub, self._bus, "", bias, old=self.bu0, wgt=self.wgt_u)
            self.paracel_bupdate_multi(self.kib, self._bis, "", bias, old=self.bi0, wgt=self.wgt_i)
            self.iter_commit()
            self._push_done = torch.cuda.Event()
            self._push_done.record(self._push_stream)

    def round(self) -> RoundResult:
        """One round: pull (or wait for) the rows, one SGD pass over the local ratings, push, commit.
        Everything is queued on the current stream; the returned handle gives the pass's squared
        error once its copy has arrived."""
        with self.phase("pull_or_wait"):
            if self._push_done is not None and self.paracel_would_pull(self.kW, self.Wl):
                # the pull must see this rank's own pushes
                torch.cuda.current_stream(self.device).wait_event(self._push_done)
            self.read_mf_paras()
        with self.phase("sgd"):
            self.sse.zero_()
            self.sgd_pass()
        slot = self._res_no % self.RESULT_SLOTS
        self._res_no += 1
        self._sse_host[slot].copy_(self.sse, non_blocking=True)
        self._sse_ev[slot].record()
        result = RoundResult(self._sse_ev[slot], self._sse_host[slot], self, self._res_no)
        if self.overlap_push and self.world > 1 and self.ssp and self.staleness >= 2:
            self._push_overlapped()
        else:
            self._push_sync()
        if self.metrics is not None:
            rows = self.lu.numel() + self.li.numel()
            self.log_metrics(round=self.clock, ratings=self.nnz, rows_held=rows,
                             bytes_pulled=rows * (self.D + 1) * 4, bytes_pushed=rows * (self.D + 1) * 4,
                             h2d_bytes=self.h2d_bytes, staleness=self.staleness,
                             sse_of_pass=result.sse() if self.metrics_sync else None)
        return result

    def phase_times_ms(self):
        """Mean device time of each phase of round() over the rounds run since ``phase_timing``
        was switched on (synchronises)."""
        summ = self.phase_summary()
        rounds = int(summ.get("sgd", {}).get("count", 0))
        out: Dict[str, float] = {k: v["ms"] / max(rounds, 1) for k, v in summ.items()}
        out["rounds"] = rounds
        return out

    def checkpoint_extra(self):
        return {"mu": self.mu, "total_nnz": self.total_nnz}

    def restore_extra(self, extra):
        self.mu, self.total_nnz = float(extra["mu"]), int(extra["total_nnz"])

    def fit(self):
        """Run the rounds that are left (all of them, or the rest after ``load_checkpoint``)."""
        for _ in range(self.clock, self.rounds):
            self.round()
        self.paracel_sync()
        self.paracel_check()
        self.pull(fused_wait=False)
        self.paracel_sync()

    def solve(self):
        """``init_parameters`` + ``learning`` of the reference's solve() (mf.hpp:325-335); the
        ratings must have been loaded with ``load_ratings``."""
        self.init_parameters()
        self.set_total_iters(self.rounds)
        self.paracel_sync()
        self.fit()

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

    def heldout_sse(self, u: torch.Tensor, i: torch.Tensor, r: torch.Tensor, chunk: int = 1 << 18):
        """Sum of squared errors of the clipped estimate on (user, item, rating) triples this
        rank has not trained on.  The rows come from their owners' shards through
        ``paracel_read_multi`` (any id, not only the rows this rank holds).  Returns
        ``(sse, count)`` as Python floats; all-reduce them for the global RMSE."""
        dev = self.device
        u, i = u.to(dev, torch.int64), i.to(dev, torch.int64)
        r = r.to(dev, torch.float32)
        sse = torch.zeros((), dtype=torch.float64, device=dev)
        for s0 in range(0, u.numel(), chunk):
            uu, ii = u[s0:s0 + chunk].contiguous(), i[s0:s0 + chunk].contiguous()
            W = self.paracel_read_multi(self.paracel_keys(self.W_tab, uu), ssp_wait=False, use_cache=False)
            H = self.paracel_read_multi(self.paracel_keys(self.H_tab, ii), ssp_wait=False, use_cache=False)
            bu = self.paracel_read_multi(self.paracel_keys(self.ub_tab, uu), ssp_wait=False, use_cache=False)
            bi = self.paracel_read_multi(self.paracel_keys(self.ib_tab, ii), ssp_wait=False, use_cache=False)
            pred = (self.mu + bu + bi + (W * H).sum(1)).clamp_(1.0, 5.0)
            sse += ((pred - r[s0:s0 + chunk]).double() ** 2).sum()
        return float(sse.item()), float(u.numel())

    # ------------------------------------------------------------------ dump
    def dump_result(self, outdir: str = "", user_names=None, item_names=None):
        """Write miu_0, ubias_0, ibias_0, W_0, H_0 in the reference's text layout
        (mf.hpp:380-492).  As there, worker 0 reads each kind of key with its filter
        (``paracel_read_special``; the rows come out of the owners' HBM over NVLink) and writes
        them.  The ids printed are those of the key names; ``user_names`` / ``item_names``
        (arrays indexed by row) rename them when the tables were built without names."""
        from ..utils.dump import dump_dict_scalar, dump_dict_vector
        outdir = outdir or self.output
        self.paracel_sync()
        if self.rank == 0:
            os.makedirs(outdir, exist_ok=True)
            dump_dict_scalar({"miu": self.mu, "rating_sz": float(self.total_nnz)},
                             os.path.join(outdir, "miu_0"))

            def ident(key, user):
                j = int(key.rsplit("_", 1)[1])
                tab = user_names if user else item_names
                own = self.user_names if user else self.item_names
                return j if (tab is None or own is not None) else int(tab[j])
            for fname, flt, user in (("ubias_0", "mf_ubias_filter", True), ("ibias_0", "mf_ibias_filter", False)):
                d = self.paracel_read_special("", flt)
                dump_dict_scalar({ident(k_, user): v for k_, v in d.items()}, os.path.join(outdir, fname))
            for fname, flt, user in (("W_0", "mf_W_filter", True), ("H_0", "mf_H_filter", False)):
                d = self.paracel_read_special("", flt)
                dump_dict_vector({ident(k_, user): v[: self.k] for k_, v in d.items()},
                                 os.path.join(outdir, fname))
        self.paracel_sync()

    def free(self):
        self.Wt = self.Ht = self.but = self.bit = None
        self.close()
