"""Vertex-centric (Pregel-style) layer on top of ``paralg`` (reference:
include/pregel/vertex.hpp:29-145).

A subclass implements ``compute(neighbor, wgt, val)`` -- what an active vertex sends along
one out-edge, normally a ``paracel_bupdate`` of the neighbour's key -- and
``mutable_value(msg)`` -- how the combined message read back from the server becomes the
vertex's new value.  ``run_supersteps`` alternates compute over the active vertices, a
barrier, ``vote_to_halt`` (a vertex whose value did not change goes inactive) and an
all-reduce of the halt flags, until every worker reports that nothing was active."""
from __future__ import annotations

import inspect
from typing import Any, Callable, Dict

from .graph import digraph
from .load.parser import parser_a
from .paralg import paralg


class vertex:
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "",
                 parser: Callable = parser_a, init_func: Callable = None, **kw):
        self.pt = paralg(hosts_dct_str, comm, output, **kw)
        self.grp = digraph()
        self.pt.paracel_load_as_graph(self.grp, input, parser, "fmap", numeric=False)
        self.vertex_val_map: Dict[str, Any] = {}
        self.vertex_adj_edge_val_map: Dict[str, Dict[str, float]] = {}
        self.vertex_active_map: Dict[str, bool] = {}
        self.init_vars(init_func or (lambda vid: float(vid)))

    def init_vars(self, func: Callable) -> None:
        nargs = len(inspect.signature(func).parameters)
        if nargs >= 3:
            self.grp.traverse(lambda r, c, w: self.vertex_val_map.__setitem__(r, func(r, c, w)))
        else:
            for v, nb in self.grp.adj.items():
                if nb:
                    self.vertex_val_map[v] = func(v)
        for v in self.vertex_val_map:
            self.vertex_adj_edge_val_map[v] = self.grp.adjacent(v)
            self.vertex_active_map[v] = True

    def compute(self, neighbor: str, wgt: float, val: Any) -> None:  # pragma: no cover
        raise NotImplementedError

    def mutable_value(self, msg: Any) -> Any:  # pragma: no cover
        raise NotImplementedError

    def vote_to_halt(self) -> None:
        for vtx in self.vertex_active_map:
            old = self.vertex_val_map[vtx]
            new = self.mutable_value(self.pt.paracel_read(vtx, default=old))
            self.vertex_val_map[vtx] = new
            self.vertex_active_map[vtx] = (old != new)

    def run_supersteps(self) -> int:
        steps = 0
        while True:
            halt_flag = 1
            for vtx, active in self.vertex_active_map.items():
                if active:
                    halt_flag = 0
                    for nb, w in self.vertex_adj_edge_val_map[vtx].items():
                        self.compute(nb, w, self.vertex_val_map[vtx])
            self.pt.paracel_sync()
            self.vote_to_halt()
            steps += 1
            if self.pt.get_comm().allreduce(halt_flag) == self.pt.get_worker_size():
                break
            self.pt.paracel_sync()
        self.pt.paracel_sync()
        return steps

    def dump_result(self, prefix: str) -> None:
        self.pt.paracel_dump_dict(dict(self.vertex_val_map), prefix)


class max_vertex_value_pregel(vertex):
    """The reference's Pregel example (max_vertex_value_pregel.cpp:28-53)."""

    def __init__(self, *a, update_file: str = "", **kw):
        self.update_file = update_file
        super().__init__(*a, **kw)
        # superstep 0: every vertex publishes its own value
        for v, val in self.vertex_val_map.items():
            self.pt.paracel_bupdate(v, val, self.update_file, "max_updater")
        self.pt.paracel_sync()

    def compute(self, neighbor, wgt, val):
        self.pt.paracel_bupdate(neighbor, val, self.update_file, "max_updater")

    def mutable_value(self, msg):
        return float(msg)
