"""Steady-state inversion on a bipartite graph (reference:
tool/steady_state_inversion_serial.cpp:40-261).

Left nodes (ids ending in ``L``) carry a distribution ``pl``, right nodes (ending in ``R``) a
target distribution ``pr`` and a score.  A walker at left node i moves to right node j with
probability ``w_ij s_j / sum_j' w_ij' s_j'``.  While some right node receives less than
``pr_j (1 - epsilon)``, its score is re-solved by Newton iterations on
``sum_i pl_i a_i x / (a_i x + c_i) = pr_j (1 - delta)``.  Output: ``score_0`` and the top-100
transition probabilities per left node in ``transfer_prob_matrix_0``."""
from __future__ import annotations

from typing import Dict, Optional

from ..graph import bigraph
from ..utils.ext import str_split
from ..utils.misc import json_parser
from ._common import cli, serial_paralg

EPSILON = 1e-4
DELTA = EPSILON / 2
KTOP = 100


class steady_state_inversion:
    def __init__(self, bigraph_input: str, dis_input: str, output: str):
        self.pt = serial_paralg(output)
        self.bigraph_input, self.dis_input = bigraph_input, dis_input
        self.score: Dict[str, float] = {}
        self.pl: Dict[str, float] = {}
        self.pr: Dict[str, float] = {}

    def trans_prob(self, i: str, j: str) -> float:
        row = self.G.adj.get(i, {})
        if j not in row:
            return 0.0
        s = sum(w * self.score[jj] for jj, w in row.items())
        return row[j] * self.score[j] / s if s else 0.0

    def q(self, r: str) -> float:
        return sum(p * self.trans_prob(i, r) for i, p in self.pl.items())

    def q_solve(self, r: str) -> float:
        AC = {}
        for i in self.pl:
            row = self.G.adj.get(i, {})
            if r in row:
                AC[i] = (row[r], sum(w * self.score[s] for s, w in row.items() if s != r))
        L = self.pr[r] * (1 - DELTA)
        x = self.score[r]
        for _ in range(100):
            f = fp = 0.0
            for i, (a, c) in AC.items():
                c2 = a * x + c
                if c2 == 0:
                    continue
                f += self.pl[i] * a * x / c2
                fp += self.pl[i] * a * c / (c2 * c2)
            f -= L
            if abs(f) <= 1e-10 or fp == 0:
                break
            x -= f / fp
            if x != x:
                break
        return x

    def solve(self):
        self.G = bigraph()
        self.pt.paracel_load_as_graph(self.G, self.bigraph_input, lambda l: str_split(l, ","), "fmap",
                                      numeric=False)
        for line in self.pt.paracel_loadall(self.dis_input):
            if not line:
                continue
            k, v = str_split(line, ",")[:2]
            self.score[k] = float(v)
            (self.pl if k.endswith("L") else self.pr)[k] = float(v)
        for t in range(20):
            new = {}
            for j, pj in self.pr.items():
                left = self.q(j)
                if left != 0.0 and left < pj * (1 - EPSILON):
                    new[j] = self.q_solve(j)
            self.score.update(new)
            if not new:
                break
        self.score_new = {k: v for k, v in self.score.items() if k.endswith("R")}
        self.transfer = {}
        for i in self.pl:
            lst = [(j[:-1], self.trans_prob(i, j)) for j in self.pr]
            lst = sorted([x for x in lst if x[1] > 0], key=lambda x: -x[1])[:KTOP]
            if lst:
                self.transfer[i[:-1]] = lst

    def dump_result(self):
        self.pt.paracel_dump_dict(self.score_new, "score_")
        self.pt.paracel_dump_prob_mtx(self.transfer, "transfer_prob_matrix_")


def solve_files(bigraph_input: str, dis_input: Optional[str], output: str):
    s = steady_state_inversion(bigraph_input, dis_input or bigraph_input, output)
    s.solve()
    s.dump_result()
    return s


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    solve_files(pt.check_parse("bigraph_input", str), pt.check_parse("distribution_input", str),
                pt.parse("output", str))


if __name__ == "__main__":
    raise SystemExit(cli(main))
