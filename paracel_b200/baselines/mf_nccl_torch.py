"""NCCL-only PyTorch baseline of the MF-SGD round: the same pull / local SGD / push structure as
``MfSgdGpu`` written with stock PyTorch ops and NCCL collectives only (``all_to_all_single`` for
the keyed pull and push, ``index_select`` / ``index_add_`` for gather and scatter-add, minibatch
SGD with per-row averaging for the local pass).  This is the baseline the fused kernels are
measured against, not a product path."""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..utils.decomp import npfact2d


class MfSgdNcclTorch:
    def __init__(self, n_users, n_items, k=128, alpha=0.005, beta=0.02, rounds=1, staleness=0, ssp=False,
                 group=None, device=None, seed=0, batch=1 << 20, **_):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.nu, self.ni, self.k, self.D = n_users, n_items, k, k
        self.alpha, self.beta, self.seed, self.batch = alpha, beta, seed, batch
        self.npx, self.npy = npfact2d(self.world)
        w = self.world
        g = torch.Generator(device=self.device)
        g.manual_seed(seed * 1000003 + self.rank)
        self.Wt = 0.1 * torch.rand((n_users + w - 1) // w, k, device=self.device, generator=g)
        self.Ht = 0.1 * torch.rand((n_items + w - 1) // w, k, device=self.device, generator=g)
        self.but = 0.1 * torch.rand((n_users + w - 1) // w, device=self.device, generator=g)
        self.bit = 0.1 * torch.rand((n_items + w - 1) // w, device=self.device, generator=g)
        self.sse = torch.zeros(1, dtype=torch.float64, device=self.device)

        class _Clock:
            def check(self_inner):
                return None
        self.clock = _Clock()

    # keyed pull / push through all_to_all
    def _plan(self, ids):
        owner = ids % self.world
        order = torch.argsort(owner, stable=True)
        counts = torch.bincount(owner, minlength=self.world)
        rc = torch.empty_like(counts)
        if self.world > 1:
            dist.all_to_all_single(rc, counts, group=self.group)
        else:
            rc = counts.clone()
        send_ids = (ids[order] // self.world).contiguous()
        recv_ids = torch.empty(int(rc.sum()), dtype=torch.int64, device=self.device)
        if self.world > 1:
            dist.all_to_all_single(recv_ids, send_ids, rc.tolist(), counts.tolist(), group=self.group)
        else:
            recv_ids = send_ids
        return {"order": order, "counts": counts.tolist(), "rc": rc.tolist(), "recv_ids": recv_ids}

    def _pull(self, table, plan):
        rows = table.index_select(0, plan["recv_ids"]).contiguous()
        out = torch.empty((len(plan["order"]),) + tuple(table.shape[1:]), device=self.device)
        if self.world > 1:
            dist.all_to_all_single(out, rows, plan["counts"], plan["rc"], group=self.group)
        else:
            out = rows
        res = torch.empty_like(out)
        res[plan["order"]] = out
        return res

    def _push(self, table, plan, delta):
        send = delta[plan["order"]].contiguous()
        recv = torch.empty((len(plan["recv_ids"]),) + tuple(table.shape[1:]), device=self.device)
        if self.world > 1:
            dist.all_to_all_single(recv, send, plan["rc"], plan["counts"], group=self.group)
        else:
            recv = send
        table.index_add_(0, plan["recv_ids"], recv)

    def load_ratings(self, u, i, r, keep_on_host=False):
        dev = self.device
        u, i, r = u.to(dev, torch.int64), i.to(dev, torch.int64), r.to(dev, torch.float32)
        self.nnz = u.numel()
        self.lu, self.ru = torch.unique(u, return_inverse=True)
        self.li, self.ri = torch.unique(i, return_inverse=True)
        perm = torch.randperm(self.nnz, device=dev)
        self.ru, self.ri, self.rr = self.ru[perm], self.ri[perm], r[perm]
        self._sum_r = float(r.sum(dtype=torch.float64))
        self.plan_u, self.plan_i = self._plan(self.lu), self._plan(self.li)

    def init_parameters(self):
        tot = torch.tensor([self._sum_r, float(self.nnz)], dtype=torch.float64, device=self.device)
        if self.world > 1:
            dist.all_reduce(tot, group=self.group)
        self.mu = float(tot[0] / max(float(tot[1]), 1.0))
        self.total_nnz = int(tot[1])
        cu = torch.zeros_like(self.but)
        ci = torch.zeros_like(self.bit)
        self._push(cu, self.plan_u, torch.ones(self.lu.numel(), device=self.device))
        self._push(ci, self.plan_i, torch.ones(self.li.numel(), device=self.device))
        self.wgt_u = 1.0 / self._pull(cu, self.plan_u).clamp(min=1.0)
        self.wgt_i = 1.0 / self._pull(ci, self.plan_i).clamp(min=1.0)

    def round(self):
        W, H = self._pull(self.Wt, self.plan_u), self._pull(self.Ht, self.plan_i)
        bu, bi = self._pull(self.but, self.plan_u), self._pull(self.bit, self.plan_i)
        W0, H0, bu0, bi0 = W.clone(), H.clone(), bu.clone(), bi.clone()
        self.sse.zero_()
        a, b = self.alpha, self.beta
        for s in range(0, self.nnz, self.batch):
            u, i, r = self.ru[s:s + self.batch], self.ri[s:s + self.batch], self.rr[s:s + self.batch]
            wu, hi = W[u], H[i]
            pred = (self.mu + bu[u] + bi[i] + (wu * hi).sum(1)).clamp(1.0, 5.0)
            e = r - pred
            self.sse += (e.double() ** 2).sum()
            cu = torch.bincount(u, minlength=W.shape[0]).clamp(min=1).float()
            ci = torch.bincount(i, minlength=H.shape[0]).clamp(min=1).float()
            dW = a * (2 * e[:, None] * hi - b * wu) / cu[u][:, None]
            dH = a * (2 * e[:, None] * wu - b * hi) / ci[i][:, None]
            W.index_add_(0, u, dW)
            H.index_add_(0, i, dH)
            bu.index_add_(0, u, a * (2 * e - b * bu[u]) / cu[u])
            bi.index_add_(0, i, a * (2 * e - b * bi[i]) / ci[i])
        self._push(self.Wt, self.plan_u, self.wgt_u[:, None] * (W - W0))
        self._push(self.Ht, self.plan_i, self.wgt_i[:, None] * (H - H0))
        self._push(self.but, self.plan_u, self.wgt_u * (bu - bu0))
        self._push(self.bit, self.plan_i, self.wgt_i * (bi - bi0))

    def paracel_check(self):
        return None

    def heldout_sse(self, u, i, r, chunk=1 << 18):
        """Same contract as ``MfSgdGpu.heldout_sse`` (rows fetched with all_to_all); every rank
        must call it with the same number of chunks."""
        dev = self.device
        u, i, r = u.to(dev, torch.int64), i.to(dev, torch.int64), r.to(dev, torch.float32)
        sse = torch.zeros((), dtype=torch.float64, device=dev)
        for s0 in range(0, u.numel(), chunk):
            pu, pi = self._plan(u[s0:s0 + chunk]), self._plan(i[s0:s0 + chunk])
            W, H = self._pull(self.Wt, pu), self._pull(self.Ht, pi)
            bu, bi = self._pull(self.but, pu), self._pull(self.bit, pi)
            pred = (self.mu + bu + bi + (W * H).sum(1)).clamp_(1.0, 5.0)
            sse += ((pred - r[s0:s0 + chunk]).double() ** 2).sum()
        return float(sse.item()), float(u.numel())

    def running_rmse(self):
        t = self.sse.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return math.sqrt(float(t) / max(self.total_nnz, 1))

    def free(self):
        pass
