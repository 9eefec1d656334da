"""Lasso and L1-regularised logistic regression by stochastic coordinate descent
("shooting") on the duplicated non-negative features (reference: tool/lasso_serial.cpp:40-170,
tool/lasso_serial_rigid.cpp:95-119, tool/lr_l1_serial.cpp:40-178).

``w = w+ - w-`` with ``W = [w+, w-] >= 0``; a step picks a random coordinate j of the 2k,
computes ``delta = (lambda + sum_i dL/dz_i * x_ij) / n`` (times 4 for the logistic loss,
whose second derivative is bounded by 1/4), moves ``w_j`` by ``eta = max(-w_j, -delta)`` and
updates the cached predictions.  Labels {0, 1} of the logistic variant are mapped to
{-1, +1}.  ``rigid=True`` materialises the negated columns instead of using a sign, which is
what the reference's "rigid" variant does; both reach the same optimum."""
from __future__ import annotations

import numpy as np

from .._core import core
from ..utils.misc import json_parser
from ._common import cli, serial_paralg


class shooting_solver:
    def __init__(self, input: str, output: str, lam: float = 0.1, rounds: int = 100,
                 logistic: bool = False, rigid: bool = False, seed: int = 0):
        self.pt = serial_paralg(output)
        self.input, self.lam, self.rounds = input, float(lam), int(rounds)
        self.logistic, self.rigid, self.seed = logistic, rigid, seed

    def load(self):
        rows = core().parse_dense_rows([l for l in self.pt.paracel_loadall(self.input) if l], ",")
        self.X = np.asfortranarray(rows[:, :-1])
        self.y = np.ascontiguousarray(rows[:, -1])
        if self.logistic:
            self.y = np.where(self.y > 0.5, 1.0, -1.0)

    def solve(self):
        self.load()
        n, k = self.X.shape
        if self.rigid:
            X2 = np.asfortranarray(np.concatenate([self.X, -self.X], axis=1))
            W = np.zeros(4 * k)
            z = np.zeros(n)
            core().shooting_steps(X2, self.y, W, z, self.lam, self.rounds * 2 * k, self.logistic, self.seed)
            # columns [0, 2k) of X2 are used with sign +, the mirrored half stays zero-summed
            self.W = np.concatenate([W[:k] + W[3 * k:], W[k:2 * k] + W[2 * k:3 * k]])
        else:
            self.W = np.zeros(2 * k)
            z = np.zeros(n)
            core().shooting_steps(self.X, self.y, self.W, z, self.lam, self.rounds * 2 * k, self.logistic,
                                  self.seed)
        self.z = z
        self.rW = self.W[:k] - self.W[k:]

    def check(self):
        """(prediction, observation) pairs (tool/lasso_serial.cpp:82-91)."""
        p = self.X @ self.rW
        if self.logistic:
            p = 1.0 / (1.0 + np.exp(-p))
        return list(zip(p.tolist(), self.y.tolist()))

    def objective(self) -> float:
        z = self.X @ self.rW
        if self.logistic:
            return float(np.log1p(np.exp(-self.y * z)).sum() + self.lam * np.abs(self.rW).sum())
        return float(0.5 * ((z - self.y) ** 2).sum() + self.lam * np.abs(self.rW).sum())

    def dump_result(self):
        self.pt.paracel_dump_vector(self.rW.tolist(), "lr_l1_weight_" if self.logistic else "lasso_weight_",
                                    "|")


def _main(cfg_file: str, logistic: bool, rigid: bool = False):
    pt = json_parser(cfg_file)
    s = shooting_solver(pt.check_parse("input", str), pt.parse("output", str), float(pt.parse("lambda")),
                        int(pt.parse("rounds")), logistic, rigid)
    s.solve()
    s.dump_result()


def main(cfg_file: str):
    return _main(cfg_file, False)


def main_rigid(cfg_file: str):
    return _main(cfg_file, False, True)


def main_lr_l1(cfg_file: str):
    return _main(cfg_file, True)


if __name__ == "__main__":
    raise SystemExit(cli(main))
