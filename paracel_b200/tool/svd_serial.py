"""Serial truncated SVD (reference: tool/svd_serial.cpp:48-154), written on numpy / scipy only so
that it is an oracle for the parallel ``models/svd.py`` and the device ``models/svd_gpu.py``
that shares no code with them.

Stages, as in the reference: (1) rank-k factorisation ``A ~ W H^T`` by alternating least squares
on the normal equations (``W = A H (H^T H)^-1``, ``H = A^T W (W^T W)^-1``; the reference runs ten
sweeps); (2) Cholesky-QR of both factors (``M^T M = L L^T``, ``Q = M L^-T``, ``R = L^T``);
(3) SVD of the small ``k x k`` core ``R_W R_H^T``; then ``U = Q_W U_core``, ``V = Q_H V_core``.
Input lines are ``row,col,value``; output files ``SIGMA_0`` (one line), ``U_0`` and ``V_0``
(``id<TAB>v1|v2|...``)."""
from __future__ import annotations

import numpy as np

from ..utils.ext import str_split
from ..utils.misc import json_parser
from ._common import cli, serial_paralg


class svd_serial:
    def __init__(self, input: str, output: str, k: int, iters: int = 10, seed: int = 0):
        self.pt = serial_paralg(output)
        self.input, self.k, self.iters, self.seed = input, int(k), int(iters), int(seed)
        self.row_ids, self.col_ids = [], []
        self.sigma = self.U = self.V = None

    def _load(self):
        import scipy.sparse as sp
        rows, cols, vals = [], [], []
        rmap, cmap = {}, {}
        for line in self.pt.paracel_loadall(self.input):
            f = str_split(line, ",")
            if len(f) < 3:
                continue
            rows.append(rmap.setdefault(f[0], len(rmap)))
            cols.append(cmap.setdefault(f[1], len(cmap)))
            vals.append(float(f[2]))
        self.row_ids, self.col_ids = list(rmap), list(cmap)
        return sp.csr_matrix((vals, (rows, cols)), shape=(len(rmap), len(cmap)), dtype=np.float64)

    @staticmethod
    def _chol_qr(M):
        L = np.linalg.cholesky(M.T @ M)
        return np.linalg.solve(L, M.T).T, L.T          # Q = M L^-T, R = L^T

    def solve(self):
        A = self._load()
        rng = np.random.default_rng(self.seed)
        H = rng.uniform(-1.0, 1.0, (A.shape[1], self.k))
        W = None
        for _ in range(self.iters):
            W = np.linalg.solve(H.T @ H, (A @ H).T).T
            H = np.linalg.solve(W.T @ W, (A.T @ W).T).T
        self.residual = float(np.sqrt(((A.toarray() - W @ H.T) ** 2).mean())) if A.shape[0] * A.shape[1] <= 1 << 22 else None
        qw, rw = self._chol_qr(W)
        qh, rh = self._chol_qr(H)
        u, s, vt = np.linalg.svd(rw @ rh.T)
        self.sigma, self.U, self.V = s, qw @ u, qh @ vt.T
        return self

    def dump_result(self):
        self.pt.paracel_dump_vector(self.sigma.tolist(), "SIGMA_")
        self.pt.paracel_dump_dict({r: self.U[i].tolist() for i, r in enumerate(self.row_ids)}, "U_")
        self.pt.paracel_dump_dict({c: self.V[j].tolist() for j, c in enumerate(self.col_ids)}, "V_")


def solve(input: str, output: str, k: int, iters: int = 10, seed: int = 0) -> svd_serial:
    s = svd_serial(input, output, k, iters=iters, seed=seed).solve()
    s.dump_result()
    return s


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    solve(pt.check_parse("input", str), pt.parse("output", str), pt.parse("k", int))


if __name__ == "__main__":
    raise SystemExit(cli(main))
