"""Steady-state inversion on a bipartite graph, parallel over the left nodes.

The reference ships this algorithm as a serial tool only (tool/steady_state_inversion_serial.cpp:
40-261); its parallel class is an empty stub (alg/misc/steady_state_inversion/
steady_state_inversion.hpp:51-57).  This class runs the same iteration on the parameter server:

* the edges ``left,right,weight`` are partitioned by left node (``fmap``), so every worker holds
  complete rows; the two distributions (left ``pl``, target ``pr``) are read by everybody;
* the scores of the right nodes live under the key ``ssi_score`` (one vector); a sweep computes
  every worker's share of ``q_j = sum_i pl_i w_ij s_j / sum_j' w_ij' s_j'`` and adds it into
  ``ssi_q_<t>``;
* the right nodes that receive less than ``pr_j (1 - epsilon)`` are re-solved together by Newton
  steps on ``sum_i pl_i a_i x / (a_i x + c_i) = pr_j (1 - delta)``: per step every worker adds
  its share of ``f`` and ``f'`` for all of them into one key, the step is taken from the sums, and
  a node stops once ``|f| <= 1e-10`` (the serial tool's rule, node by node);
* like the serial tool the sweep is Jacobi (all deficits of a sweep are solved against the scores
  at its start) and stops after 20 sweeps or when no node is short.

Output (rank 0): ``score_0``; every worker: ``transfer_prob_matrix_<rank>`` with the 100 largest
transition probabilities of its left nodes.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

from ..paralg import paralg
from ..utils.ext import str_split

EPSILON = 1e-4
DELTA = EPSILON / 2
KTOP = 100
SWEEPS = 20
NEWTON_STEPS = 100


class steady_state_inversion(paralg):
    def __init__(self, comm, hosts_dct_str, input: str = "", output: str = "",
                 distribution_input: str = "", **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input = input
        self.dis_input = distribution_input or input
        self.sweeps = 0

    # ------------------------------------------------------------------ loading
    def _load(self):
        pl: Dict[str, float] = {}
        pr: Dict[str, float] = {}
        for line in self.paracel_loadall(self.dis_input):
            f = str_split(line, ",")
            if len(f) != 2:
                continue
            (pl if f[0].endswith("L") else pr)[f[0]] = float(f[1])
        self.right: List[str] = sorted(pr)
        self.pr = np.array([pr[r] for r in self.right])
        col = {r: j for j, r in enumerate(self.right)}
        rows: Dict[str, Dict[int, float]] = {}
        for line in self.paracel_load(self.input):
            f = str_split(line, ",")
            if len(f) != 3 or not f[0].endswith("L") or f[1] not in col or f[0] not in pl:
                continue
            rows.setdefault(f[0], {})[col[f[1]]] = float(f[2])
        # the lines of one left node may be split between workers' byte ranges: gather by owner
        mine: Dict[str, Dict[int, float]] = {}
        np_ = self.get_worker_size()
        if np_ > 1:
            from ..utils.hash import hash_value
            parts = [dict() for _ in range(np_)]
            for k, v in rows.items():
                parts[hash_value(k) % np_][k] = v
            for src in self.get_comm().alltoall(parts):
                for k, v in src.items():
                    mine.setdefault(k, {}).update(v)
        else:
            mine = rows
        self.left = sorted(mine)
        self.pl = np.array([pl[i] for i in self.left])
        ri, ci, w = [], [], []
        for a, i in enumerate(self.left):
            for j, x in sorted(mine[i].items()):
                ri.append(a); ci.append(j); w.append(x)
        self.ri = np.array(ri, dtype=np.int64)
        self.ci = np.array(ci, dtype=np.int64)
        self.w = np.array(w, dtype=np.float64)

    # ------------------------------------------------------------------ pieces
    def _row_sums(self, score):
        s = np.zeros(len(self.left))
        np.add.at(s, self.ri, self.w * score[self.ci])
        return s

    def _local_q(self, score):
        s = self._row_sums(score)
        ok = s[self.ri] != 0
        q = np.zeros(len(self.right))
        np.add.at(q, self.ci[ok], self.pl[self.ri[ok]] * self.w[ok] * score[self.ci[ok]] / s[self.ri[ok]])
        return q

    def _sum_over_workers(self, key, vec):
        """Every worker adds its vector into ``key``; returns the total (the key is new each time)."""
        self.paracel_bupdate(key, [float(x) for x in vec], "", "add")
        self.paracel_sync()
        tot = np.array(self.paracel_read(key), dtype=np.float64)
        self.paracel_sync()
        return tot

    def _newton(self, short, score, sweep):
        """Scores of the right nodes ``short`` so that each receives ``pr_j (1 - delta)``."""
        s = self._row_sums(score)
        pos = {j: n for n, j in enumerate(short)}
        sel = np.array([c in pos for c in self.ci], dtype=bool)
        e_n = np.array([pos[c] for c in self.ci[sel]], dtype=np.int64)      # edge -> index in short
        a = self.w[sel]
        c = s[self.ri[sel]] - a * score[self.ci[sel]]
        p = self.pl[self.ri[sel]]
        x = score[short].copy()
        target = self.pr[short] * (1 - DELTA)
        live = np.ones(len(short), dtype=bool)
        for step in range(NEWTON_STEPS):
            xe = x[e_n]
            den = a * xe + c
            good = den != 0
            f = np.zeros(len(short)); fp = np.zeros(len(short))
            np.add.at(f, e_n[good], p[good] * a[good] * xe[good] / den[good])
            np.add.at(fp, e_n[good], p[good] * a[good] * c[good] / (den[good] * den[good]))
            tot = self._sum_over_workers(f"ssi_newton_{sweep}_{step}", np.concatenate([f, fp]))
            f, fp = tot[: len(short)] - target, tot[len(short):]
            live &= ~((np.abs(f) <= 1e-10) | (fp == 0))
            if not live.any():
                break
            x_new = np.where(live, x - f / np.where(fp == 0, 1.0, fp), x)
            live &= ~np.isnan(x_new)
            x = np.where(np.isnan(x_new), x, x_new)
        return x

    # ------------------------------------------------------------------ solve
    def solve(self):
        self._load()
        if self.get_worker_id() == 0:
            self.paracel_write("ssi_score", [float(x) for x in self.pr])
        self.paracel_sync()
        score = np.array(self.paracel_read("ssi_score"), dtype=np.float64)
        for t in range(SWEEPS):
            self.sweeps = t + 1
            q = self._sum_over_workers(f"ssi_q_{t}", self._local_q(score))
            short = np.nonzero((q != 0) & (q < self.pr * (1 - EPSILON)))[0]
            if short.size == 0:
                break
            score[short] = self._newton(short, score, t)
            if self.get_worker_id() == 0:
                self.paracel_write("ssi_score", [float(x) for x in score])
            self.paracel_sync()
        self.score = score
        s = self._row_sums(score)
        self.transfer = {}
        for a_, i in enumerate(self.left):
            m = self.ri == a_
            if s[a_] == 0:
                continue
            pr_ = self.w[m] * score[self.ci[m]] / s[a_]
            lst = sorted(((self.right[j][:-1], float(v)) for j, v in zip(self.ci[m], pr_) if v > 0),
                         key=lambda x: -x[1])[:KTOP]
            if lst:
                self.transfer[i[:-1]] = lst
        self.paracel_sync()

    def q(self, r: str) -> float:
        """Share of the walkers that arrive at right node ``r`` under the current scores (all workers
        must call)."""
        tot = self._sum_over_workers(f"ssi_probe_{r}_{self.sweeps}", self._local_q(self.score))
        self.sweeps += 1
        return float(tot[self.right.index(r)])

    def dump_result(self):
        if self.get_worker_id() == 0:
            self.paracel_dump_dict({r: float(v) for r, v in zip(self.right, self.score)}, "score_")
        self.paracel_dump_prob_mtx(self.transfer, "transfer_prob_matrix_")
        self.paracel_sync()
