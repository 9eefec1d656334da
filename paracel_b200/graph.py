"""Graph containers with the reference's query API (include/graph.hpp:31-744):
``undirected_graph``, ``digraph`` (with reverse adjacency), ``bigraph``,
``bigraph_continuous``, and the ``DFS`` / ``BFS`` / ``connected_components``
helpers.  Adjacency is a dict of dicts on the host (any hashable vertex id);
``to_coo`` / ``to_csr`` export the edges as tensors for the GPU kernels.  All
containers are packable (``to_packable`` / ``from_packable``) so that a graph
can be a parameter-server value, as in the sparse similarity algorithm.
"""
from __future__ import annotations

from collections import deque
from typing import Any, Callable, Dict, Hashable, Iterable, List, Set, Tuple

import numpy as np

from .utils.types import bag_type


class _AdjGraph:
    directed = True

    def __init__(self, edges: Any = None):
        self.adj: Dict[Hashable, Dict[Hashable, float]] = {}
        self.e_sz = 0
        if edges is None:
            return
        if isinstance(edges, dict):
            self.construct_from_dict(edges)
        else:
            edges = list(edges)
            if edges and len(edges[0]) == 2:
                self.construct_from_tuples(edges)
            else:
                self.construct_from_triples(edges)

    def construct_from_dict(self, edge_info: Dict) -> None:
        for v, nb in edge_info.items():
            for w, wgt in nb.items():
                self.add_edge(v, w, wgt)

    def construct_from_tuples(self, tpls: Iterable[Tuple]) -> None:
        for v, w in tpls:
            self.add_edge(v, w)

    def construct_from_triples(self, tpls: Iterable[Tuple]) -> None:
        for v, w, wgt in tpls:
            self.add_edge(v, w, wgt)

    def add_edge(self, v, w, wgt: float = 1.0) -> None:
        raise NotImplementedError

    def get_data(self) -> Dict:
        return self.adj

    def traverse(self, *args) -> None:
        """``traverse(func)`` visits every edge as func(v, w, wgt); ``traverse(v, func)``
        visits the edges leaving ``v``."""
        if len(args) == 1:
            func = args[0]
            for v, nb in self.adj.items():
                for w, wgt in nb.items():
                    func(v, w, wgt)
        else:
            v, func = args
            for w, wgt in self.adj.get(v, {}).items():
                func(v, w, wgt)

    def traverse_by_vertex(self, func: Callable) -> None:
        """Call ``func((vertex, {neighbour: weight}))`` once per vertex: like the reference, which
        hands ``func`` the ``std::pair`` of its adjacency map (graph.hpp:104-108, 255-259), the
        argument is the (vertex, adjacency) pair, not the bare vertex."""
        for item in self.adj.items():
            func(item)

    def v(self) -> int:
        return len(self.adj)

    def e(self) -> int:
        return self.e_sz

    def adjacent(self, v) -> Dict[Hashable, float]:
        return dict(self.adj.get(v, {}))

    def vertex_bag(self) -> List:
        return list(self.adj.keys())

    def vertex_set(self) -> Set:
        return set(self.adj.keys())

    def outdegree(self, v) -> int:
        return len(self.adj.get(v, {}))

    def degree(self, v) -> int:
        return self.outdegree(v)

    def indegree(self, vertex) -> int:
        return sum(1 for nb in self.adj.values() if vertex in nb)

    def avg_degree(self) -> float:
        return self.e() / max(self.v(), 1)

    def max_degree(self) -> int:
        return max((len(nb) for nb in self.adj.values()), default=0)

    def selfloops(self) -> int:
        return sum(1 for v, nb in self.adj.items() if v in nb)

    def dump2triples(self) -> List[Tuple]:
        return [(v, w, wgt) for v, nb in self.adj.items() for w, wgt in nb.items()]

    def dump2dict(self) -> Dict:
        return {v: dict(nb) for v, nb in self.adj.items() if nb}

    # ---- tensor exports for the device kernels
    def to_coo(self):
        """(src, dst, wgt) numpy arrays; vertex ids must be integers."""
        n = sum(len(nb) for nb in self.adj.values())
        src = np.empty(n, dtype=np.int64)
        dst = np.empty(n, dtype=np.int64)
        wgt = np.empty(n, dtype=np.float64)
        k = 0
        for v, nb in self.adj.items():
            for w, x in nb.items():
                src[k], dst[k], wgt[k] = v, w, x
                k += 1
        return src, dst, wgt

    def to_packable(self):
        return {"v_sz": self.v(), "e_sz": self.e_sz,
                "adj": [[v, [[w, x] for w, x in nb.items()]] for v, nb in self.adj.items()]}

    @classmethod
    def from_packable(cls, d):
        g = cls()
        for v, nb in d["adj"]:
            g.adj.setdefault(v, {})
            for w, x in nb:
                g.adj[v][w] = x
        g.e_sz = d["e_sz"]
        return g


class undirected_graph(_AdjGraph):
    directed = False

    def add_edge(self, v, w, wgt: float = 1.0) -> None:
        self.adj.setdefault(v, {})[w] = wgt
        self.adj.setdefault(w, {})[v] = wgt
        self.e_sz += 1


class digraph(_AdjGraph):
    def __init__(self, edges: Any = None):
        self.reverse_adj: Dict[Hashable, Dict[Hashable, float]] = {}
        super().__init__(edges)

    def add_edge(self, v, w, wgt: float = 1.0) -> None:
        self.adj.setdefault(v, {})[w] = wgt
        self.adj.setdefault(w, {})
        self.reverse_adj.setdefault(w, {})[v] = wgt
        self.e_sz += 1

    def reverse(self) -> None:
        self.adj, self.reverse_adj = self.reverse_adj, self.adj

    def reverse_adjacent(self, v) -> Dict[Hashable, float]:
        return dict(self.reverse_adj.get(v, {}))


class bigraph(_AdjGraph):
    def add_edge(self, v, w, wgt: float = 1.0) -> None:
        self.adj.setdefault(v, {})[w] = wgt
        self.e_sz += 1

    def reset(self) -> None:
        self.adj.clear()
        self.e_sz = 0

    clear = reset

    def is_connected(self, a, b) -> bool:
        return b in self.adj.get(a, {})

    def get_wgt(self, a, b) -> float:
        return self.adj[a][b]

    def traverse_by_left_vertex(self, func: Callable) -> None:
        for v in self.adj.items():
            func(v)

    def left_vertex_bag(self) -> List:
        return list(self.adj.keys())

    def left_vertex_set(self) -> Set:
        return set(self.adj.keys())


class bigraph_continuous:
    """Bipartite graph whose left vertices are the dense range 0..N-1
    (graph.hpp:514-612).  A file form ``N`` then ``src,dst,rating`` lines is accepted."""

    def __init__(self, n_or_file: Any = 0):
        self.adj: List[bag_type] = []
        self.e_sz = 0
        if isinstance(n_or_file, str):
            with open(n_or_file) as f:
                n = int(f.readline())
                self.adj = [bag_type() for _ in range(n)]
                for line in f:
                    a, b, c = line.strip().split(",")
                    self.add_edge(int(a), int(b), float(c))
        else:
            self.adj = [bag_type() for _ in range(int(n_or_file))]

    def add_edge(self, src: int, dst: int, rating: float = 1.0) -> None:
        while src >= len(self.adj):
            self.adj.append(bag_type())
        self.adj[src].put((dst, rating))
        self.e_sz += 1

    def resize(self, n: int) -> None:
        self.adj = [bag_type() for _ in range(n)]
        self.e_sz = 0

    def v(self) -> int:
        return len(self.adj)

    def e(self) -> int:
        return self.e_sz

    def adjacent(self, v: int) -> bag_type:
        return self.adj[v].get()

    def outdegree(self, v: int) -> int:
        return len(self.adj[v])

    def indegree(self, v: int) -> int:
        return sum(1 for b in self.adj for (d, _) in b if d == v)

    def traverse(self, *args) -> None:
        if len(args) == 1:
            for i, b in enumerate(self.adj):
                for d, r in b:
                    args[0](i, d, r)
        else:
            v, func = args
            for d, r in self.adj[v]:
                func(v, d, r)

    def to_packable(self):
        return {"v_sz": self.v(), "e_sz": self.e_sz,
                "adj": [[[d, r] for d, r in b] for b in self.adj]}

    @classmethod
    def from_packable(cls, d):
        g = cls(d["v_sz"])
        for i, b in enumerate(d["adj"]):
            for dst, r in b:
                g.add_edge(i, dst, r)
        return g


class DFS:
    """Depth-first traversal from ``src`` calling ``func(v)`` on first visit; records
    start/end times and the reverse post-order (graph.hpp:619-657)."""

    def __init__(self, graph, src, func: Callable = lambda v: None):
        self.marked: Dict = {}
        self.start_time: Dict = {}
        self.end_time: Dict = {}
        self.topological_order: List = []
        self.timer = 0
        # iterative to survive deep graphs
        stack = [(src, iter(graph.adjacent(src)))]
        self.marked[src] = True
        func(src)
        self.timer += 1
        self.start_time[src] = self.timer
        while stack:
            v, it = stack[-1]
            advanced = False
            for w in it:
                if w not in self.marked:
                    self.marked[w] = True
                    func(w)
                    self.timer += 1
                    self.start_time[w] = self.timer
                    stack.append((w, iter(graph.adjacent(w))))
                    advanced = True
                    break
            if not advanced:
                self.timer += 1
                self.end_time[v] = self.timer
                self.topological_order.append(v)
                stack.pop()
        self.topological_order.reverse()

    def visited(self, v) -> bool:
        return v in self.marked

    def start(self) -> Dict:
        return self.start_time

    def end(self) -> Dict:
        return self.end_time

    def torder(self) -> List:
        return self.topological_order


class BFS:
    def __init__(self, graph, src, func: Callable = lambda v: None):
        self.marked = {src: True}
        self.edge_to: Dict = {}
        self.dist_to = {src: 0}
        func(src)
        q = deque([src])
        while q:
            node = q.popleft()
            for w in graph.adjacent(node):
                if w not in self.marked:
                    self.marked[w] = True
                    func(w)
                    self.edge_to[w] = node
                    self.dist_to[w] = self.dist_to[node] + 1
                    q.append(w)

    def visited(self, v) -> bool:
        return v in self.marked

    def edgeTo(self, v):
        return self.edge_to[v]

    def dist(self, v) -> int:
        return self.dist_to[v]


class connected_components:
    def __init__(self, graph):
        self.count = 0
        self.identifier: Dict = {}
        for v in graph.vertex_bag():
            if v not in self.identifier:
                cid = self.count

                def mark(x, cid=cid):
                    self.identifier[x] = cid
                DFS(graph, v, mark)
                self.count += 1

    def is_connected(self, v, w) -> bool:
        return self.id(v) == self.id(w) and self.id(v) >= 0

    def cnt(self) -> int:
        return self.count

    def id(self, v) -> int:
        return self.identifier.get(v, -1)

    def handleCC(self, func: Callable) -> None:
        for k, c in self.identifier.items():
            func(k, c)
