"""PageRank on the host parameter server (reference: alg/graph_alg/pagerank/pr.hpp:40-200).

Input ``src,dst`` lines; a vertex without out-links appears as ``v,2147483648`` (the
sentinel target is never stored).  In-link lists ``<v>_links`` = [(src, outdeg(src))] are
built by appending through the server (concat handler), read back once, ranks start at
1/N (N = number of vertices with out-links) and each round evaluates
``pr(v) = (1-d) + d * sum pr(u)/outdeg(u)`` from a multi-read of the in-neighbours' ranks
followed by a multi-write; ranks are not re-normalised."""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..graph import digraph
from ..paralg import paralg
from ..utils.ext import str_split
from ..utils.types import SENTINEL


class pagerank(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", handle_file: str = "",
                 update_function: str = "init_updater", filter_function: str = "pr_filter",
                 rounds: int = 1, damping_factor: float = 0.85, **kw):
        super().__init__(hosts_dct_str, comm, output, rounds, **kw)
        self.input = input
        self.handle_file = handle_file
        self.update_function, self.filter_function = update_function, filter_function
        self.damping_factor = float(damping_factor)
        self.kvmap: Dict[int, float] = {}
        self.klstmap: Dict[int, List[Tuple[int, float]]] = {}

    def init_paras(self):
        self.local_graph = digraph()
        self.paracel_load_as_graph(self.local_graph, self.input, lambda l: str_split(l, ","), "fmap")
        for a, nb in self.local_graph.adj.items():
            if nb:
                self.kvmap[a] = float(len(nb))
        links: Dict[int, List[Tuple[int, float]]] = {}
        for a, nb in self.local_graph.adj.items():
            for b in nb:
                links.setdefault(b, []).append((a, self.kvmap[a]))
        tmp = {f"{b}_links": [[s, d] for s, d in lst] for b, lst in links.items() if b != SENTINEL}
        if tmp:
            self.paracel_bupdate_multi(tmp, self.handle_file, self.update_function)
        self.paracel_sync()
        self.klstmap = {}
        for v in self.kvmap:
            got = self.paracel_read(f"{v}_links", default=[])
            self.klstmap[v] = [(int(s), float(d)) for s, d in got]
        node_sz = self.get_comm().allreduce(len(self.kvmap))
        init_val = 1.0 / max(node_sz, 1)
        for v in self.kvmap:
            self.kvmap[v] = init_val
        self.paracel_write_multi({f"{v}_pr": init_val for v in self.kvmap})
        self.paracel_sync()

    def learning(self):
        need = sorted({s for lst in self.klstmap.values() for s, _ in lst})
        keys = [f"{s}_pr" for s in need]
        d = self.damping_factor
        self.paracel_sync()
        for rd in range(self.rounds):
            vals = self.paracel_read_multi(keys) if keys else []
            stale = dict(zip(need, vals))
            for v, lst in self.klstmap.items():
                sigma = sum(stale[s] / od for s, od in lst)
                self.kvmap[v] = (1.0 - d) + d * sigma
            self.paracel_sync()
            self.paracel_write_multi({f"{v}_pr": r for v, r in self.kvmap.items()})
            self.paracel_sync()
        allv = self.paracel_read_special(self.handle_file, self.filter_function)
        self.kvmap = {int(k.split("_")[0]): float(v) for k, v in allv.items()}

    def solve(self):
        self.init_paras()
        self.paracel_sync()
        self.learning()

    def dump_result(self):
        if self.get_worker_id() == 0:
            self.paracel_dump_dict({str(k): v for k, v in self.kvmap.items()}, "pagerank_")
