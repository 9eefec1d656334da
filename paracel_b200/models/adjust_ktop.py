"""Per-user neighbourhood size for similarity-weighted rating prediction (reference:
alg/recommendation/adjust_ktop_sparse/adjust_ktop_sparse.hpp:36-200).

The similarity graph ``id\\tid:sim|id:sim`` is model-partitioned (``fset``), ratings
``u,i,r`` are published as scalar keys ``<uid>_<iid>`` and looked up with the tolerant
multi-read; for every user the neighbours are added in decreasing similarity and the k that
minimises the squared residual of ``sum s_uv a_vi / sum s_uv`` is kept."""
from __future__ import annotations

import math
from typing import Dict

from ..graph import bigraph
from ..paralg import paralg
from ..utils.ext import str_split


class adjust_ktop_s(paralg):
    def __init__(self, comm, hosts_dct_str, rating_input: str, fmt: str, sim_input: str,
                 low_limit: int = 1, output: str = "", **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.rating_input, self.fmt, self.sim_input = rating_input, fmt, sim_input
        self.low_limit = max(int(low_limit), 1)
        self.ktop_result: Dict[int, int] = {}
        self.training_rmse = 0.0
        self.original_rmse = 0.0

    def solve(self):
        def sim_parser(line):
            tmp = str_split(line, "\t")
            return [tmp[0]] + str_split(tmp[1], "|")
        self.sim_G = bigraph()
        self.paracel_load_as_graph(self.sim_G, self.sim_input, sim_parser, "fset")

        def rp(line):
            return str_split(line, ",")

        def rp_sfv(line):
            t = str_split(line, ",")
            return [t[1], t[0], t[2]]
        self.rating_G = bigraph()
        self.paracel_load_as_graph(self.rating_G, self.rating_input,
                                   rp_sfv if self.fmt == "sfv" else rp, "fmap")
        msg = {f"{u}_{i}": v for u, nb in self.rating_G.adj.items() for i, v in nb.items()}
        if msg:
            self.paracel_write_multi(msg)
        self.paracel_sync()
        for uid in self.sim_G.left_vertex_set():
            self.ktop_result[uid] = self.linear_search(uid)
        self.paracel_sync()

    def linear_search(self, node) -> int:
        ktop_list = sorted(self.sim_G.adjacent(node).items(), key=lambda kv: -kv[1])
        mine = self.rating_G.adjacent(node)
        if not mine:  # ratings of this user live on another worker: read them
            mine = {int(k.split("_")[1]): v for k, v in
                    self.paracel_read_special("", f"prefix:{node}_").items()}
        ktop, res_min, flag = -1, float("inf"), False
        N: Dict[int, float] = {}
        Dn: Dict[int, float] = {}
        for idx in range(self.low_limit - 1, len(ktop_list)):
            v, suv = ktop_list[idx]
            keys = [f"{v}_{i}" for i in mine]
            vals = self.paracel_read_multi(keys, as_dict=True) if keys else {}
            residual = 0.0
            for i, aui in mine.items():
                avi = vals.get(f"{v}_{i}")
                if avi is not None:
                    N[i] = N.get(i, 0.0) + avi * suv
                    Dn[i] = Dn.get(i, 0.0) + suv
                if N and Dn.get(i, 0.0) != 0:
                    residual += (aui - N[i] / Dn[i]) ** 2
            if idx == len(ktop_list) - 1:
                self.original_rmse += residual
            if not flag or residual < res_min:
                if not flag and residual == 0:
                    continue
                ktop, res_min, flag = idx + 1, residual, True
        if ktop == -1:
            return len(ktop_list)
        self.training_rmse += res_min
        return ktop

    def _rmse(self, s: float) -> float:
        tot = self.worker_comm.allreduce([s, float(self.rating_G.e())])
        return math.sqrt(tot[0] / max(tot[1], 1.0))

    def cal_rmse(self) -> float:
        return self._rmse(self.training_rmse)

    def cal_original_rmse(self) -> float:
        return self._rmse(self.original_rmse)

    def dump_result(self):
        self.paracel_dump_dict({str(k): int(v) for k, v in self.ktop_result.items()}, "ktop_result_")
