"""Full-batch gradient-descent logistic regression (reference: tool/lr_serial.cpp:40-218)."""
from __future__ import annotations

import numpy as np

from .._core import core
from ..utils.misc import json_parser
from ._common import cli, serial_paralg


class lr_serial:
    def __init__(self, input: str, output: str, rounds: int = 100, alpha: float = 0.01,
                 beta: float = 0.0, seed: int = 0):
        self.pt = serial_paralg(output)
        self.input, self.rounds, self.alpha, self.beta = input, rounds, alpha, beta
        self.rng = np.random.default_rng(seed)

    def solve(self):
        rows = core().parse_dense_rows([l for l in self.pt.paracel_loadall(self.input) if l], ",")
        y = np.ascontiguousarray(rows[:, -1])
        X = np.ascontiguousarray(np.concatenate([np.ones((rows.shape[0], 1)), rows[:, :-1]], 1))
        n, d = X.shape
        theta = self.rng.random(d)
        for _ in range(self.rounds):
            h = 1.0 / (1.0 + np.exp(-X @ theta))
            theta = theta + self.alpha * (X.T @ (y - h)) / n - 2 * self.alpha * self.beta * theta
        self.theta, self.X, self.y = theta, X, y

    def loss(self) -> float:
        return core().logloss_sum(self.X, self.y, np.ascontiguousarray(self.theta)) / max(len(self.y), 1)

    def dump_result(self):
        self.pt.paracel_dump_vector(self.theta.tolist(), "lr_theta_", "|")


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    s = lr_serial(pt.check_parse("input", str), pt.parse("output", str), int(pt.get("rounds", 100)),
                  float(pt.get("alpha", 0.01)), float(pt.get("beta", 0.0)))
    s.solve()
    print("loss:", s.loss())
    s.dump_result()


if __name__ == "__main__":
    raise SystemExit(cli(main))
