"""One half-iteration of alternating least squares (reference:
alg/recommendation/als/als.hpp:40-330, als_driver.cpp, als_validate_driver.cpp).

Given fixed item factors H (file ``id\\tf1|f2|...``) every user's factor is the ridge
solution ``(H_u^T H_u + lambda I)^-1 H_u^T a_u`` over the items the user rated.  Ratings
``u,i,r`` are loaded with pattern ``fmap`` (train user factors) or ``smap``.  The host path
solves with LAPACK; ``device=True`` uses the batched normal-equation + Cholesky kernel
(``csrc/cuda/als.cu``).  ``validate`` sweeps a list of lambdas and reports train / validation
RMSE like the reference's validate driver."""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np

from ..graph import bigraph
from ..paralg import paralg
from ..utils.ext import str_split


class alternating_least_square_standard(paralg):
    def __init__(self, comm, hosts_dct_str, rating_input: str, factor_input: str, output: str = "",
                 pattern: str = "fmap", lam: float = 0.1, device: bool = False, **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.rating_input, self.factor_input = rating_input, factor_input
        self.pattern, self.lam, self.device = pattern, float(lam), device
        self.W: Dict[int, List[float]] = {}
        self.H: Dict[int, np.ndarray] = {}
        self.kdim = 0

    def load(self):
        self.rating_graph = bigraph()
        self.paracel_load_as_graph(self.rating_graph, self.rating_input, lambda l: str_split(l, ","),
                                   self.pattern)
        need = {b for nb in self.rating_graph.adj.values() for b in nb}

        def take(lines):
            for line in lines:
                if not line:
                    continue
                v = str_split(line, "\t")
                iid = int(v[0])
                fac = str_split(v[1], "|")
                self.kdim = len(fac)
                if iid in need:
                    self.H[iid] = np.asarray([float(x) for x in fac])
        self.paracel_sequential_loadall(self.factor_input, take)

    def learning(self):
        users = sorted(self.rating_graph.adj.keys())
        if not users:
            return
        if self.device:
            self._learning_device(users)
            return
        I = np.eye(self.kdim)
        for uid in users:
            nb = self.rating_graph.adj[uid]
            try:
                Hs = np.stack([self.H[b] for b in nb])
            except KeyError as e:
                raise RuntimeError("Data error: rating data and factor data is not consistent.") from e
            ai = np.asarray(list(nb.values()))
            self.W[uid] = np.linalg.solve(Hs.T @ Hs + self.lam * I, Hs.T @ ai).tolist()

    def _learning_device(self, users):
        import torch
        from ..ops.als import als_solve
        items = sorted(self.H.keys())
        pos = {b: j for j, b in enumerate(items)}
        Hm = torch.tensor(np.stack([self.H[b] for b in items]), dtype=torch.float32, device="cuda")
        ptr, idx, val = [0], [], []
        for uid in users:
            nb = self.rating_graph.adj[uid]
            idx.extend(pos[b] for b in nb)
            val.extend(nb.values())
            ptr.append(len(idx))
        Wm = als_solve(torch.tensor(ptr, dtype=torch.int64, device="cuda"),
                       torch.tensor(idx, dtype=torch.int32, device="cuda"),
                       torch.tensor(val, dtype=torch.float32, device="cuda"), Hm, self.lam)
        Wm = Wm.cpu().tolist()
        for uid, w in zip(users, Wm):
            self.W[uid] = w

    def solve(self):
        self.load()
        self.learning()

    def estimate(self, uid, iid) -> float:
        return float(np.dot(self.W[uid], self.H[iid]))

    def cal_rmse(self) -> float:
        s = 0.0
        for uid, nb in self.rating_graph.adj.items():
            for iid, r in nb.items():
                e = r - self.estimate(uid, iid)
                s += e * e
        tot = self.worker_comm.allreduce([s, float(self.rating_graph.e())])
        return math.sqrt(tot[0] / max(tot[1], 1.0))

    def validate(self, validate_input: str, lambdas: Sequence[float]):
        """For every lambda: solve, then (train RMSE, validation RMSE over pairs whose user and
        item are known to this worker)."""
        self.load()
        vlines = [l for l in self.paracel_load(validate_input) if l]
        out = []
        for lam in lambdas:
            self.lam = float(lam)
            self.learning()
            train = self.cal_rmse()
            s, n = 0.0, 0
            for line in vlines:
                a, b, r = str_split(line, ",")[:3]
                uid, iid = int(a), int(b)
                if uid in self.W and iid in self.H:
                    e = float(r) - self.estimate(uid, iid)
                    s += e * e
                    n += 1
            tot = self.worker_comm.allreduce([s, float(n)])
            out.append((lam, train, math.sqrt(tot[0] / max(tot[1], 1.0))))
        return out

    def dump_result(self):
        self.paracel_dump_dict({str(k): v for k, v in self.W.items()}, "W_")
