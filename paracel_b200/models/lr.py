"""Logistic regression on the parameter server (reference:
alg/classification/logistic_regression/lr.cpp:40-365, lr_driver.cpp:26-80).

Four learning methods, all on one dense key ``theta`` (bias first):

* ``dgd``      full pass with theta frozen, accumulated step pushed once per round;
* ``ipm``      iterative parameter mixing: local sequential SGD pass, push
               ``(theta - theta_pulled) / n_workers`` (default);
* ``downpour`` pull every n/800 samples, push every n/1000 samples;
* ``agd``      pull and push around every sample.

The per-sample step is ``theta_i += alpha (y - sigmoid(theta.x)) x_i - 2 alpha beta theta_i``.
Unlike the reference, whose LR constructor hard-wires SSP off (lr.cpp:55-56),
``limit_s`` / ``ssp_switch`` are exposed; with SSP on, rounds are committed with
``iter_commit`` and the two barriers per round are dropped.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from .._core import core
from ..paralg import paralg
from ..utils.ext import str_split


class logistic_regression(paralg):
    logistic = True
    theta_prefix = "lr_theta_"
    default_handler = "lr_theta_update"

    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", update_file: str = "",
                 update_func: str = "", method: str = "ipm", rounds: int = 1, alpha: float = 0.002,
                 beta: float = 0.1, debug: bool = False, limit_s: int = 0, ssp_switch: bool = False,
                 seed: Optional[int] = None, **kw):
        super().__init__(hosts_dct_str, comm, output, rounds, limit_s, ssp_switch, **kw)
        self.input = input
        self.update_file = update_file
        self.update_func = update_func or self.default_handler
        self.learning_method = method
        self.worker_id = self.worker_comm.get_rank()
        self.alpha, self.beta, self.debug = float(alpha), float(beta), bool(debug)
        self.kdim = 0
        self.loss_error: List[float] = []
        self.predv: List[Tuple[List[float], float]] = []
        self.theta = np.zeros(0)
        self.rng = np.random.default_rng(seed if seed is not None else None)
        self.samples = np.zeros((0, 0))
        self.labels = np.zeros(0)

    # ---------------------------------------------------------------- data
    def local_parser(self, lines: Sequence[str], sep: str = ","):
        """``f1,...,fk,label`` -> rows [1, f1..fk] and labels."""
        rows = core().parse_dense_rows([l for l in lines if l], sep)
        if rows.shape[0] == 0:
            self.samples = np.zeros((0, max(self.kdim, 0) + 1))
            self.labels = np.zeros(0)
            return
        self.labels = np.ascontiguousarray(rows[:, -1])
        self.samples = np.ascontiguousarray(
            np.concatenate([np.ones((rows.shape[0], 1)), rows[:, :-1]], axis=1))
        if self.kdim == 0:
            self.kdim = self.samples.shape[1] - 1

    def hypothesis(self, X: np.ndarray) -> np.ndarray:
        z = X @ self.theta
        return 1.0 / (1.0 + np.exp(-z)) if self.logistic else z

    # ------------------------------------------------------------ learning
    def _init_theta(self, dim: int):
        self.theta = self.rng.random(dim)
        self.paracel_write("theta", self.theta.tolist())  # every worker writes; last writer wins
        self.paracel_register_bupdate(self.update_file, self.update_func)

    def _pass(self, idx: np.ndarray, theta: np.ndarray, delta: np.ndarray, accumulate: bool):
        core().linear_sgd_pass(self.samples, self.labels, np.ascontiguousarray(idx, dtype=np.int64),
                               theta, delta, self.alpha, self.beta, self.logistic, accumulate)

    def _round_end(self):
        if self.ssp_switch:
            self.iter_commit()
        else:
            self.paracel_sync()

    def _learn(self, method: str):
        n, dim = self.samples.shape
        self._init_theta(dim)
        if self.ssp_switch:
            self.paracel_sync()  # everybody has written before anybody reads
        idx = np.arange(n, dtype=np.int64)
        wgt = 1.0 / self.get_worker_size()
        read_batch = max(n // 800, 1) if n // 800 else 10
        update_batch = max(n // 1000, 1) if n // 1000 else 10
        for rd in range(self.rounds):
            self.rng.shuffle(idx)
            theta = np.ascontiguousarray(self.paracel_read("theta"), dtype=np.float64)
            delta = np.zeros(dim)
            if method == "dgd":
                self._pass(idx, theta, delta, True)
                if not self.ssp_switch:
                    self.paracel_sync()
                self.paracel_bupdate("theta", delta.tolist())
                self._round_end()
            elif method == "ipm":
                theta_old = theta.copy()
                self._pass(idx, theta, delta, False)
                if not self.ssp_switch:
                    self.paracel_sync()
                self.paracel_bupdate("theta", (wgt * (theta - theta_old)).tolist())
                self._round_end()
            elif method == "downpour":
                theta_old = theta.copy()
                start = 0
                while start < n:
                    if start % read_batch == 0 or start == n - 1:
                        theta = np.ascontiguousarray(self.paracel_read("theta"), dtype=np.float64)
                        theta_old = theta.copy()
                    stop = min(n, start + update_batch)
                    self._pass(idx[start:stop], theta, delta, False)
                    self.paracel_bupdate("theta", (theta - theta_old).tolist())
                    theta_old = theta.copy()
                    start = stop
                self._round_end()
            elif method == "agd":
                for s in idx:
                    theta = np.ascontiguousarray(self.paracel_read("theta"), dtype=np.float64)
                    theta_old = theta.copy()
                    self._pass(np.asarray([s]), theta, delta, False)
                    self.paracel_bupdate("theta", (theta - theta_old).tolist())
                if self.ssp_switch:
                    self.iter_commit()
            else:
                raise ValueError(f"method {method!r} is not supported")
            self.theta = theta
            if self.debug:
                self.loss_error.append(self.calc_loss())
        if self.ssp_switch:
            self.paracel_sync()
        self.theta = np.asarray(self.paracel_read("theta"), dtype=np.float64)  # last pull

    def dgd_learning(self):
        self._learn("dgd")

    def ipm_learning(self):
        self._learn("ipm")

    def downpour_learning(self):
        self._learn("downpour")

    def agd_learning(self):
        self._learn("agd")

    def solve(self):
        import time
        t0 = time.time()
        lines = self.paracel_load(self.input)
        self.local_parser(lines)
        self.paracel_sync()
        t1 = time.time()
        self._learn(self.learning_method)
        self.paracel_sync()
        # wall-clock seconds of the two phases (load + parse, learning rounds)
        self.seconds_load, self.seconds_learn = t1 - t0, time.time() - t1

    # ------------------------------------------------------------- metrics
    def calc_loss(self) -> float:
        """Mean log-loss over all workers' samples (lr.cpp:321-336)."""
        loss = core().logloss_sum(self.samples, self.labels, np.ascontiguousarray(self.theta)) \
            if self.samples.shape[0] else 0.0
        loss = self.worker_comm.allreduce(float(loss))
        sz = self.worker_comm.allreduce(int(self.samples.shape[0]))
        return loss / max(sz, 1)

    def test(self, test_fn: str) -> float:
        self.local_parser(self.paracel_load(test_fn))
        loss = self.calc_loss()
        self.paracel_sync()
        return loss

    def predict(self, pred_fn: str):
        lines = [l for l in self.paracel_load(pred_fn) if l]
        self.predv = []
        for line in lines:
            f = [float(x) for x in str_split(line, ",")[: self.kdim]]
            x = np.asarray([1.0] + f)
            self.predv.append((x.tolist(), float(self.hypothesis(x[None, :])[0])))
        self.paracel_sync()

    def dump_result(self):
        if self.worker_id == 0:
            self.paracel_dump_vector(self.theta.tolist(), self.theta_prefix, "|")
            if self.debug:
                self.paracel_dump_vector(self.loss_error, "lr_loss_error_", "\n")
        self.paracel_dump_vector(self.predv, "pred_v_", "\n")


class ridge_regression(logistic_regression):
    """Ridge regression by ipm SGD with squared loss (reference:
    alg/regression/ridge/ridge.hpp:33-130); same structure as LR with h = theta.x."""
    logistic = False
    theta_prefix = "ridge_theta_"
    default_handler = "ridge_theta_update"

    def calc_loss(self) -> float:
        r = self.samples @ self.theta - self.labels if self.samples.shape[0] else np.zeros(0)
        loss = self.worker_comm.allreduce(float((r * r).sum()))
        sz = self.worker_comm.allreduce(int(self.samples.shape[0]))
        return loss / max(sz, 1)
