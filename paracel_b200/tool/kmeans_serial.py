"""Serial k-means on ``id\\tf1,f2,...`` rows (reference: tool/kmeans_serial.cpp:40-139)."""
from __future__ import annotations

import numpy as np

from ..utils.ext import str_split
from ..utils.misc import json_parser
from ._common import cli, serial_paralg


class kmeans_serial:
    def __init__(self, input: str, output: str, kclusters: int, rounds: int):
        self.pt = serial_paralg(output)
        self.input, self.k, self.rounds = input, int(kclusters), int(rounds)

    def solve(self):
        ids, rows = [], []
        for line in self.pt.paracel_loadall(self.input):
            if line:
                a, b = str_split(line, "\t")
                ids.append(a)
                rows.append([float(x) for x in str_split(b, ",")])
        X = np.asarray(rows)
        C = X[: self.k].copy()
        owner = np.zeros(len(ids), dtype=np.int64)
        for _ in range(self.rounds):
            d2 = (C * C).sum(1)[None, :] - 2 * X @ C.T
            owner = d2.argmin(1)
            for c in range(self.k):
                if (owner == c).any():
                    C[c] = X[owner == c].mean(0)
        self.clusters = C
        self.groups = {c: [ids[i] for i in np.nonzero(owner == c)[0]] for c in range(self.k)}

    def dump_result(self):
        self.pt.paracel_dump_dict({k: v for k, v in self.groups.items() if v}, "kmeans_")
        self.pt.paracel_dump_dict({i: c.tolist() for i, c in enumerate(self.clusters)}, "centers_")


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    s = kmeans_serial(pt.check_parse("input", str), pt.parse("output", str), pt.parse("kclusters", int),
                      pt.parse("rounds", int))
    s.solve()
    s.dump_result()


if __name__ == "__main__":
    raise SystemExit(cli(main))
