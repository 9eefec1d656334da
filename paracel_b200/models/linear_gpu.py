"""Linear models on GPUs with the weight vector in a ``DenseTable`` (device path of the
reference's logistic / ridge regression, alg/classification/logistic_regression/lr.cpp, and
the parameter-server form of its serial L1 tools, tool/lr_l1_serial.cpp, tool/lasso_serial.cpp).

Both classes are ``paralg`` subclasses on the device backend; the weights are the dense key
``"theta"``.  One step is the reference's "dgd" round (lr.cpp:119-145) on a minibatch:

    theta = paracel_read("theta")            all-gather of the shards by peer loads
    g     = sum_rows (y - h(theta.x)) x      dense / sparse gradient kernel, written into
                                             paracel_delta_buffer("theta")
    paracel_bupdate("theta", g, "", handler, collective=True)
                                             reduce-scatter fused with the handler at the owner

with handler ``sgd`` (plain step), ``prox_l1`` (proximal gradient: soft threshold with
lambda -- sparse L1 logistic regression / Lasso) or ridge's shrinkage folded into the step.
``DenseLinearGpu`` also has the reference's asynchronous methods (lr.cpp:154-299): ``ipm``
(local SGD pass, then one update with the mean of the workers' moves), ``downpour`` and ``agd``
(local SGD with one-sided pushes of the accumulated move and periodic re-reads), whose updates
are one-sided reductions into the owners' HBM (``paracel_update``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.linear import DenseGrad, sparse_grad
from ..paralg import paralg


def remap_by_frequency(cols: torch.Tensor, n_features: int):
    """Renumber features by decreasing frequency (the hottest get the smallest ids, which the
    sparse gradient kernel keeps in shared memory).  Returns (new cols, old id of each new id)."""
    cnt = torch.bincount(cols.long(), minlength=n_features)
    order = torch.argsort(cnt, descending=True, stable=True)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(n_features, device=cols.device)
    return inv[cols.long()].to(torch.int32), order


class SparseLinearGpu(paralg):
    def __init__(self, n_features: int, eta: float = 0.5, lam: float = 1e-6, logistic: bool = True,
                 l1: bool = True, group=None, device=None, hot_T: int = 8192, nbatch: int = 1,
                 comm=None, hosts_dct_str=None, output: str = ""):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.group = group
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.F, self.eta, self.lam, self.logistic = int(n_features), float(eta), float(lam), logistic
        self.handler = "prox_l1" if l1 else "sgd"
        self.table = self.paracel_dense_table("theta", self.F, handler=self.handler).table
        self.table.count_nnz = True
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
        # the gradient kernel indexes theta with these column ids: check them once
        _lib.validate_ids(self.cols, 0, self.F, "sparse linear model (feature ids)")
        self.paracel_write("theta", torch.zeros(self.F, device=dev))

    def step(self):
        """One minibatch step on every rank; returns nothing (loss stays on the device)."""
        lo, hi = self.batches[self.step_no % self.nbatch]
        self.step_no += 1
        theta = self.paracel_read("theta")
        delta = self.paracel_delta_buffer("theta")
        delta.zero_()
        self.loss.zero_()
        if hi > lo:
            base = self.row_ptr[lo:hi + 1]
            # the kernel indexes cols/vals with absolute offsets taken from row_ptr
            sparse_grad(base, self.cols, self.vals, self.y[lo:hi], theta, delta, self.loss,
                        self.logistic, self.hot_T)
        nb = self.n_total / self.nbatch
        self.paracel_bupdate("theta", delta, "", self.handler, collective=True, lr=-self.eta / nb,
                             lam=self.lam)

    def epoch(self):
        with self.phase("epoch"):
            for _ in range(self.nbatch):
                self.step()
        self.log_metrics(step=self.step_no, samples=self.n_local)

    def checkpoint_extra(self):
        return {"step_no": self.step_no}

    def restore_extra(self, extra):
        self.step_no = int(extra["step_no"])

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
        return self.paracel_read("theta").clone()

    def free(self):
        self.table = None
        self.close()


class DenseLinearGpu(paralg):
    """Dense logistic / ridge regression, one ``dgd`` round per step."""

    def __init__(self, dim: int, eta: float = 0.1, beta: float = 0.0, logistic: bool = True,
                 group=None, device=None, comm=None, hosts_dct_str=None, output: str = ""):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.group = group
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.d, self.eta, self.beta, self.logistic = int(dim), float(eta), float(beta), logistic
        self.table = self.paracel_dense_table("theta", self.d, handler="sgd").table
        self.grad = DenseGrad(self.d, self.device)

    def load(self, X: torch.Tensor, y: torch.Tensor, theta0: Optional[torch.Tensor] = None):
        self.X = X.to(self.device, torch.float32).contiguous()
        self.y = y.to(self.device, torch.float32).contiguous()
        n = torch.tensor([self.y.numel()], dtype=torch.int64, device=self.device)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        self.n_total = int(n.item())
        # collective write: the first read on any rank waits until every owner holds its slice
        self.paracel_write("theta", theta0 if theta0 is not None else torch.zeros(self.d, device=self.device))

    def step(self):
        theta = self.paracel_read("theta")
        delta = self.paracel_delta_buffer("theta")
        self.grad(self.X, self.y, theta, delta, self.logistic)
        if self.beta:
            # ridge / L2 shrinkage of the reference's update rule: - 2 alpha beta theta per sample
            delta.add_(theta, alpha=-2.0 * self.beta * self.y.numel())
        self.paracel_bupdate("theta", delta, "", "sgd", collective=True, lr=-self.eta / self.n_total)

    # ------------------------------------------------ asynchronous methods (lr.cpp:154-299)
    def _local_sgd(self, theta: torch.Tensor, lo: int, hi: int, alpha: float, batch: int):
        """Minibatch SGD over rows [lo, hi) on a private copy of theta (the reference steps
        sample by sample; a minibatch of ``batch`` rows is one gradient kernel here)."""
        g = self._async_g
        for b0 in range(lo, hi, batch):
            b1 = min(hi, b0 + batch)
            self.grad(self.X[b0:b1], self.y[b0:b1], theta, g, self.logistic)
            theta.mul_(1.0 - 2.0 * alpha * self.beta * (b1 - b0) / batch)
            theta.add_(g, alpha=alpha / (b1 - b0))
        return theta

    def fit_async(self, method: str = "ipm", rounds: int = 1, alpha: float = 0.05, batch: int = 4096,
                  pull_every: int = 8, push_every: int = 10):
        """``ipm``: every round each worker runs SGD from the shared theta over its rows and
        the mean of the workers' moves is applied (one update per worker and round).
        ``downpour``: SGD on a private copy; every ``push_every`` minibatches the accumulated
        move is pushed one-sidedly (divided by the worker count) and every ``pull_every``
        minibatches theta is read again, with no synchronisation between workers.
        ``agd``: read and push around every minibatch."""
        if method not in ("ipm", "downpour", "agd"):
            raise ValueError("method must be ipm, downpour or agd")
        n, W = self.y.numel(), self.world
        self._async_g = torch.empty(self.d, device=self.device)
        if method == "agd":
            pull_every = push_every = 1
        for _ in range(rounds):
            theta = self.paracel_read("theta").clone()
            base = theta.clone()
            if method == "ipm":
                self._local_sgd(theta, 0, n, alpha, batch)
                self.paracel_update("theta", (theta - base) / W, "", "lr_theta_update").result()
                self.paracel_sync()
                continue
            nb = 0
            for b0 in range(0, n, batch):
                self._local_sgd(theta, b0, min(n, b0 + batch), alpha, batch)
                nb += 1
                if nb % push_every == 0:
                    self.paracel_update("theta", (theta - base) / W, "", "lr_theta_update")
                    base.copy_(theta)
                if nb % pull_every == 0:
                    move = theta - base          # keep what has not been pushed yet
                    theta = self.paracel_read("theta").clone()
                    base = theta.clone()
                    theta.add_(move)
            self.paracel_update("theta", (theta - base) / W, "", "lr_theta_update").result()
            self.paracel_sync()

    def mean_loss(self) -> float:
        t = self.grad.loss.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return float(t.item()) / max(self.n_total, 1)

    def weights(self) -> torch.Tensor:
        return self.paracel_read("theta").clone()

    def free(self):
        self.table = None
        self.close()
