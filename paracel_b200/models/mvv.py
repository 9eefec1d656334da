"""Max-vertex-value: every vertex ends with the largest value reachable along in-edges
(reference: alg/graph_alg/max_vertex_value/max_vertex_value.hpp:40-140).  Vertex values
start as the numeric vertex id; active vertices push their value to their out-neighbours
with the ``max`` handler until no value changes anywhere."""
from __future__ import annotations

from typing import Dict

from ..graph import digraph
from ..paralg import paralg
from ..utils.ext import str_split


class max_vertex_value(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", update_file: str = "",
                 update_func: str = "max_updater", **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input, self.update_file, self.update_func = input, update_file, update_func
        self.vertex_val_map: Dict[str, float] = {}
        self.active: Dict[str, bool] = {}

    def init(self):
        self.grp = digraph()
        self.paracel_load_as_graph(self.grp, self.input, lambda l: str_split(l, ","), "fmap",
                                   numeric=False)
        for v, nb in self.grp.adj.items():
            if nb:  # owned vertices are the ones with out-links on this worker
                self.vertex_val_map[v] = float(v)
                self.active[v] = True
        self.out = {v: list(self.grp.adj[v].keys()) for v in self.vertex_val_map}

    def solve(self):
        self.init()
        for v, val in self.vertex_val_map.items():
            self.paracel_bupdate(v, val, self.update_file, self.update_func)
        self.paracel_sync()
        while True:
            halt = 1
            for v, act in self.active.items():
                if act:
                    halt = 0
                    for w in self.out[v]:
                        self.paracel_bupdate(w, self.vertex_val_map[v], self.update_file,
                                             self.update_func)
            self.paracel_sync()
            for v in self.active:
                new = float(self.paracel_read(v))
                self.active[v] = new != self.vertex_val_map[v]
                self.vertex_val_map[v] = new
            self.paracel_sync()
            if self.get_comm().allreduce(halt) == self.get_worker_size():
                break
            self.paracel_sync()
        self.paracel_sync()

    def dump_result(self):
        self.paracel_dump_dict(dict(self.vertex_val_map), "vertex_val_")
