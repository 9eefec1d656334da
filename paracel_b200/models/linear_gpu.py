"""Linear models on GPUs with the weight vector in a ``DenseTable`` (device path of the
reference's logistic / ridge regression, alg/classification/logistic_regression/lr.cpp, and
the parameter-server form of its serial L1 tools, tool/lr_l1_serial.cpp, tool/lasso_serial.cpp).

One step is the reference's "dgd" round (lr.cpp:119-145) on a minibatch:

    theta = paracel_read("theta")            -> DenseTable.read    (all-gather by peer loads)
    g     = sum_rows (y - h(theta.x)) x      -> dense / sparse gradient kernel, written into
                                                 the table's delta buffer
    paracel_bupdate("theta", g)              -> DenseTable.bupdate (reduce-scatter fused with the
                                                 registered handler)

with handler ``sgd`` (plain step), ``prox_l1`` (proximal gradient: soft threshold with
lambda -- sparse L1 logistic regression / Lasso) or ridge's shrinkage folded into the step.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops.linear import DenseGrad, sparse_grad
from ..ps.tables import DenseTable


def remap_by_frequency(cols: torch.Tensor, n_features: int):
    """Renumber features by decreasing frequency (the hottest get the smallest ids, which the
    sparse gradient kernel keeps in shared memory).  Returns (new cols, old id of each new id)."""
    cnt = torch.bincount(cols.long(), minlength=n_features)
    order = torch.argsort(cnt, descending=True, stable=True)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(n_features, device=cols.device)
    return inv[cols.long()].to(torch.int32), order


class SparseLinearGpu:
    def __init__(self, n_features: int, eta: float = 0.5, lam: float = 1e-6, logistic: bool = True,
                 l1: bool = True, group=None, device=None, hot_T: int = 8192, nbatch: int = 1):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.F, self.eta, self.lam, self.logistic = int(n_features), float(eta), float(lam), logistic
        self.table = DenseTable(self.F, group, device, handler="prox_l1" if l1 else "sgd")
        self.device = self.table.device
        self.hot_T, self.nbatch = hot_T, max(1, int(nbatch))
        self.loss = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.step_no = 0

    def load(self, row_ptr: torch.Tensor, cols: torch.Tensor, y: torch.Tensor,
             vals: Optional[torch.Tensor] = None):
        """This rank's rows as CSR (int64 row_ptr, int32 cols, optional fp32 vals) and labels."""
        dev = self.device
        self.row_ptr = row_ptr.to(dev, torch.int64).contiguous()
        self.cols = cols.to(dev, torch.int32).contiguous()
        self.vals = None if vals is None else vals.to(dev, torch.float32).contiguous()
        self.y = y.to(dev, torch.float32).contiguous()
        self.n_local = self.y.numel()
        n = torch.tensor([self.n_local], dtype=torch.int64, device=dev)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        self.n_total = int(n.item())
        # minibatch boundaries in rows
        b = torch.linspace(0, self.n_local, self.nbatch + 1).long().tolist()
        self.batches = [(b[i], b[i + 1]) for i in range(self.nbatch)]
        self.table.write(torch.zeros(self.F, device=dev))

    def step(self):
        """One minibatch step on every rank; returns nothing (loss stays on the device)."""
        lo, hi = self.batches[self.step_no % self.nbatch]
        self.step_no += 1
        theta = self.table.read()
        delta = self.table.delta()
        delta.zero_()
        self.loss.zero_()
        if hi > lo:
            base = self.row_ptr[lo:hi + 1]
            # the kernel indexes cols/vals with absolute offsets taken from row_ptr
            sparse_grad(base, self.cols, self.vals, self.y[lo:hi], theta, delta, self.loss,
                        self.logistic, self.hot_T)
        nb = self.n_total / self.nbatch
        self.table.bupdate(lr=-self.eta / nb, lam=self.lam, count_nnz=True)

    def epoch(self):
        for _ in range(self.nbatch):
            self.step()

    def mean_loss(self) -> float:
        """Mean loss of the last step's minibatch (before that step's update), all ranks."""
        t = self.loss.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return float(t.item()) / max(self.n_total / self.nbatch, 1.0)

    def nnz_weights(self) -> int:
        t = self.table.nnz.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return int(t.item())

    def weights(self) -> torch.Tensor:
        return self.table.read().clone()

    def free(self):
        torch.cuda.synchronize(self.device)
        self.table.free()


class DenseLinearGpu:
    """Dense logistic / ridge regression, one ``dgd`` round per step."""

    def __init__(self, dim: int, eta: float = 0.1, beta: float = 0.0, logistic: bool = True,
                 group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.d, self.eta, self.beta, self.logistic = int(dim), float(eta), float(beta), logistic
        self.table = DenseTable(self.d, group, device, handler="sgd")
        self.device = self.table.device
        self.grad = DenseGrad(self.d, self.device)

    def load(self, X: torch.Tensor, y: torch.Tensor, theta0: Optional[torch.Tensor] = None):
        self.X = X.to(self.device, torch.float32).contiguous()
        self.y = y.to(self.device, torch.float32).contiguous()
        n = torch.tensor([self.y.numel()], dtype=torch.int64, device=self.device)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        self.n_total = int(n.item())
        self.table.write(theta0 if theta0 is not None else torch.zeros(self.d, device=self.device))

    def step(self):
        theta = self.table.read()
        delta = self.table.delta()
        self.grad(self.X, self.y, theta, delta, self.logistic)
        if self.beta:
            # ridge / L2 shrinkage of the reference's update rule: - 2 alpha beta theta per sample
            delta.add_(theta, alpha=-2.0 * self.beta * self.y.numel())
        self.table.bupdate(lr=-self.eta / self.n_total)

    def mean_loss(self) -> float:
        t = self.grad.loss.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return float(t.item()) / max(self.n_total, 1)

    def weights(self) -> torch.Tensor:
        return self.table.read().clone()

    def free(self):
        torch.cuda.synchronize(self.device)
        self.table.free()
