"""One half-iteration of alternating least squares on GPUs (device path of
alg/recommendation/als/als.hpp:40-330).

``AlsGpu`` is a ``paralg`` subclass on the device backend.  The fixed item factors are the rows
``H_<iid>`` of a table sharded over the ranks' HBM (every rank writes the part of the factor
file it read to the owners); the users are partitioned over the ranks as by the reference's
``fmap`` pattern (als.hpp:174).  ``solve`` is

    H_local = paracel_read_multi(keys of the items my users rated)     sparse keyed pull over NVLink
    W       = batched normal equations + Cholesky, one CTA per user    csrc/cuda/als.cu
    paracel_write_multi(keys of my users, W)                           rows W_<uid> to their owners

so no rank ever holds all of H, unlike the host path, which streams the whole factor file
through every worker (als.hpp:103-131).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops.als import als_solve
from ..paralg import paralg


class AlsGpu(paralg):
    def __init__(self, n_users: int, n_items: int, k: int, lam: float = 0.1, group=None, device=None,
                 comm=None, hosts_dct_str=None, output: str = "", user_names=None, item_names=None):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.group = group
        self.n_users, self.n_items, self.k, self.lam = int(n_users), int(n_items), int(k), float(lam)
        self.kp = (self.k + 3) // 4 * 4
        self.user_names, self.item_names = user_names, item_names
        self.H_tab = self.paracel_row_table(self.n_items, self.kp, prefix="H_", names=item_names)
        self.W_tab = self.paracel_row_table(self.n_users, self.kp, prefix="W_", names=user_names)

    def _pad(self, M: torch.Tensor) -> torch.Tensor:
        if M.shape[1] == self.kp:
            return M.contiguous()
        out = torch.zeros(M.shape[0], self.kp, device=self.device)
        out[:, : M.shape[1]] = M
        return out

    def load(self, u: torch.Tensor, i: torch.Tensor, r: torch.Tensor,
             item_rows: Optional[torch.Tensor] = None, item_factors: Optional[torch.Tensor] = None):
        """``(u, i, r)``: the ratings of the users this rank solves for (table rows).
        ``item_rows`` / ``item_factors``: the slice of the factor file this rank read; it is
        written to the owners of those rows."""
        dev = self.device
        if item_rows is not None and item_rows.numel():
            self.paracel_write_multi(self.paracel_keys(self.H_tab, item_rows.to(dev, torch.int64)),
                                     self._pad(item_factors.to(dev, torch.float32)))
        self.paracel_sync()
        u, i = u.to(dev, torch.int64), i.to(dev, torch.int64)
        self.lu, ru = torch.unique(u, return_inverse=True)
        self.li, ri = torch.unique(i, return_inverse=True)
        order = torch.argsort(ru, stable=True)
        self.ru, self.ri = ru[order], ri[order].to(torch.int32).contiguous()
        self.rr = r.to(dev, torch.float32)[order].contiguous()
        self.ptr = torch.zeros(self.lu.numel() + 1, dtype=torch.int64, device=dev)
        self.ptr[1:] = torch.cumsum(torch.bincount(self.ru, minlength=self.lu.numel()), 0)
        self.kH = self.paracel_keys(self.H_tab, self.li)
        self.kW = self.paracel_keys(self.W_tab, self.lu)
        self.W = torch.zeros(self.lu.numel(), self.k, device=dev)

    def solve(self, lam: Optional[float] = None):
        if lam is not None:
            self.lam = float(lam)
        if self.lu.numel():
            self.Hl = self.paracel_read_multi(self.kH, use_cache=False)[:, : self.k].contiguous()
            self.W = als_solve(self.ptr, self.ri, self.rr, self.Hl, self.lam)
            self.paracel_write_multi(self.kW, self._pad(self.W))
        else:
            self.Hl = torch.zeros(0, self.k, device=self.device)
        self.paracel_sync()
        self.paracel_check()

    def cal_rmse(self) -> float:
        t = torch.zeros(2, dtype=torch.float64, device=self.device)
        if self.rr.numel():
            pred = (self.W[self.ru] * self.Hl[self.ri.long()]).sum(1)
            t[0] = ((pred - self.rr).double() ** 2).sum()
            t[1] = self.rr.numel()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return math.sqrt(float(t[0]) / max(float(t[1]), 1.0))

    def validate_sse(self, u: torch.Tensor, i: torch.Tensor, r: torch.Tensor):
        """(sse, count) over validation triples given as table rows; rows come from the tables."""
        dev = self.device
        if u.numel() == 0:
            return 0.0, 0.0
        W = self.paracel_read_multi(self.paracel_keys(self.W_tab, u.to(dev, torch.int64)), use_cache=False)
        H = self.paracel_read_multi(self.paracel_keys(self.H_tab, i.to(dev, torch.int64)), use_cache=False)
        e = (W * H).sum(1) - r.to(dev, torch.float32)
        return float((e.double() ** 2).sum().item()), float(u.numel())

    def dump_result(self, outdir: str = ""):
        """``W_<rank>``: ``uid\\tf1|f2|...`` for the users this rank solved (als.hpp:316-318)."""
        from ..utils.dump import dump_dict_vector
        outdir = outdir or self.output
        os.makedirs(outdir, exist_ok=True)
        ids = self.lu.cpu().tolist()
        if self.user_names is not None:
            ids = [int(self.user_names[j]) for j in ids]
        dump_dict_vector(dict(zip((str(x) for x in ids), self.W.cpu().tolist())),
                         os.path.join(outdir, f"W_{self.rank}"))
        self.paracel_sync()

    def free(self):
        self.close()
