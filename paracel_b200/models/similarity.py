"""Cosine similarity top-k (reference: alg/recommendation/similarity_dense/sim_dense.hpp:60-200,
ab_sim_dense, and alg/recommendation/similarity_sparse/sim_sparse_row.hpp:40-200).

``sim_dense``: rows ``id,f1,...,fk`` of input_a are normalised and compared against every
block of input_b (the whole file streamed block by block); per item the ``ktop`` most
similar other items with similarity >= ``simbar`` are kept.  With ``device=True`` each
block product runs on the tcgen05 tf32 GEMM (3xTF32) and the top-k selection on the GPU.

``sim_sparse_row``: rows of a bipartite graph (``row,col,val`` or swapped with fmt ``sfv``)
are normalised, every worker publishes its block as one graph-valued parameter ``G_<rank>``
and then walks the other workers' blocks in ring order ``(rank + i) % W``."""
from __future__ import annotations

import heapq
from typing import Dict, List, Tuple

import numpy as np

from ..graph import bigraph
from ..paralg import paralg
from ..utils.ext import str_split


class sim_dense(paralg):
    def __init__(self, comm, hosts_dct_str, input_a: str, input_b: str = "", output: str = "",
                 simbar: float = 0.0, ktop: int = 20, device: bool = False, **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input_a, self.input_b = input_a, input_b or input_a
        self.simbar, self.ktop, self.device = float(simbar), int(ktop), device
        self.result: Dict[int, List[Tuple[int, float]]] = {}

    @staticmethod
    def _parse(lines):
        ids, rows = [], []
        for line in lines:
            if not line:
                continue
            v = str_split(line, ",")
            ids.append(int(v[0]))
            rows.append([float(x) for x in v[1:]])
        X = np.asarray(rows, dtype=np.float64) if rows else np.zeros((0, 0))
        if X.size:
            X = X / np.sqrt((X * X).sum(1, keepdims=True))
        return np.asarray(ids, dtype=np.int64), X

    def _merge(self, ids_a, ids_b, S):
        """Keep, per row of S, the ktop best columns >= simbar with a different id."""
        k = min(self.ktop, S.shape[1])
        S = np.where(ids_a[:, None] == ids_b[None, :], -np.inf, S)
        S = np.where(S >= self.simbar, S, -np.inf)
        if k <= 0:
            return
        part = np.argpartition(-S, k - 1, axis=1)[:, :k]
        for r in range(S.shape[0]):
            heap = self.heaps.setdefault(int(ids_a[r]), [])
            for c in part[r]:
                s = S[r, c]
                if s == -np.inf:
                    continue
                item = (float(s), int(ids_b[c]))
                if len(heap) < self.ktop:
                    heapq.heappush(heap, item)
                elif item > heap[0]:
                    heapq.heapreplace(heap, item)

    def solve(self):
        self.ids, self.X = self._parse(self.paracel_load(self.input_a))
        self.heaps: Dict[int, list] = {}
        if self.device:
            import torch
            from ..ops.gemm import gemm_nt
            from ..ops.misc import RunningTopK
            Xa = torch.tensor(self.X, dtype=torch.float32, device="cuda")
            topk = RunningTopK(torch.tensor(self.ids, device="cuda"), self.ktop, self.simbar)

        def handler(lines):
            ids_b, B = self._parse(lines)
            if B.shape[0] == 0 or self.X.shape[0] == 0:
                return
            if self.device:
                # GEMM tile on the tensor cores (3xTF32), top-k merge on the GPU
                Bt = torch.tensor(B, dtype=torch.float32, device="cuda")
                topk.update(gemm_nt(Xa, Bt, precise=True), torch.tensor(ids_b, device="cuda"))
                return
            self._merge(self.ids, ids_b, self.X @ B.T)
        self.paracel_sequential_loadall(self.input_b, handler)
        if self.device:
            self.result = topk.result() if self.X.shape[0] else {}
            return
        self.result = {i: [(j, s) for s, j in sorted(h, reverse=True)] for i, h in self.heaps.items()}

    def dump_result(self):
        self.paracel_dump_dict({k: v for k, v in self.result.items() if v}, "result_")


ab_sim_dense = sim_dense  # A-versus-B form: pass input_a and input_b (ab_driver.cpp)


class sim_sparse_row(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", fmt: str = "fsv",
                 topk: int = 20, sim_bar: float = 0.0, sim_ubar: float = 1.0e30, **kw):
        # rbar / cbar / rubar / cubar / weight_bar / intersect_bar / sim_method of the reference's
        # config are accepted and ignored exactly as its implementation ignores them
        for unused in ("rbar", "cbar", "rubar", "cubar", "weight_bar", "intersect_bar", "sim_method"):
            kw.pop(unused, None)
        super().__init__(hosts_dct_str, comm, output, **kw)
        if fmt not in ("fsv", "sfv"):
            raise ValueError("format parameter is invalid.")
        self.input, self.fmt, self.topk = input, fmt, int(topk)
        self.sim_bar, self.sim_ubar = float(sim_bar), float(sim_ubar)
        self.sim_result: Dict[int, list] = {}

    def normalize(self):
        for v, nb in self.G.adj.items():
            n = np.sqrt(sum(x * x for x in nb.values()))
            if n > 0:
                for w in nb:
                    nb[w] /= n

    def cal_sim(self, Gvar: bigraph):
        for var, row in self.G.adj.items():
            for other, orow in Gvar.adj.items():
                if var == other:
                    continue
                small, big = (row, orow) if len(row) <= len(orow) else (orow, row)
                sim = sum(x * big[c] for c, x in small.items() if c in big)
                if sim < self.sim_bar or sim > self.sim_ubar:
                    continue
                h = self.sim_result.setdefault(var, [])
                item = (sim, other)
                if len(h) < self.topk:
                    heapq.heappush(h, item)
                elif item > h[0]:
                    heapq.heapreplace(h, item)

    def solve(self):
        def p1(line):
            return str_split(line, ",")

        def p2(line):
            t = str_split(line, ",")
            t[0], t[1] = t[1], t[0]
            return t
        self.G = bigraph()
        self.paracel_load_as_graph(self.G, self.input, p1 if self.fmt == "fsv" else p2, "fmap")
        self.normalize()
        me, W = self.get_worker_id(), self.get_worker_size()
        self.paracel_write(f"G_{me}", self.G)
        self.paracel_sync()
        for i in range(W):
            r = (me + i) % W
            if r == me:
                self.cal_sim(self.G)
            else:
                self.cal_sim(bigraph.from_packable(self.paracel_read(f"G_{r}")))
        self.paracel_sync()

    def dump_result(self):
        res = {k: [(j, s) for s, j in sorted(h, reverse=True)] for k, h in self.sim_result.items()}
        self.paracel_dump_dict(res, "similarities_")
        self.paracel_sync()
