"""Truncated SVD by alternating least squares + Cholesky-QR + a small dense SVD (reference:
alg/recommendation/svd/svd.hpp:40-310 -- unfinished there -- and the complete serial version
tool/svd_serial.cpp:40-190).

Stage 1: rank-K factorisation A ~ W H^T by ``W = A H (H^T H)^-1``, ``H = A^T W (W^T W)^-1``
repeated ``iters`` times; A is row-partitioned over the workers, the K x K Gram matrices and
the N x K product ``A^T W`` are reduced THROUGH the parameter server (bupdate with the add
handler, barrier, read), as in svd.hpp:137-181.  Stage 2: Cholesky-QR of W and H
(``M^T M = L L^T``, ``Q = M L^-T``), SVD of the K x K matrix ``R_W R_H^T``, ``U = Q_W U_r``,
``V = Q_H V_r``.  Dumps SIGMA_0, U_<rank>, V_0."""
from __future__ import annotations


import numpy as np

from ..paralg import paralg
from ..utils.ext import str_split


class svd(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", k: int = 2,
                 update_file: str = "", update_function: str = "svd_updater", iters: int = 20,
                 oversample: int = 10, seed: int = 0, **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input, self.k = input, int(k)
        self.update_file, self.update_function = update_file, update_function
        self.iters, self.oversample, self.seed = int(iters), int(oversample), seed
        self._epoch = 0

    def _reduce(self, name: str, M: np.ndarray) -> np.ndarray:
        """All-reduce of a dense matrix through the server: add-bupdate, barrier, read."""
        self._epoch += 1
        key = f"{name}_{self._epoch}"
        self.paracel_bupdate(key, M.reshape(-1).tolist(), self.update_file, self.update_function)
        self.paracel_sync()
        out = np.asarray(self.paracel_read(key), dtype=np.float64).reshape(M.shape)
        self.paracel_sync()
        if self.get_worker_id() == 0:
            self.paracel_remove(key)
        return out

    def solve(self):
        A, rm, cm_local = self.paracel_load_as_matrix(self.input, lambda l: str_split(l, ","), "fmap")
        # global column numbering: union of the workers' column ids
        cols = sorted(set(cm_local.values()))
        allc = sorted(set().union(*self.worker_comm.allgather(cols)))
        gpos = {c: j for j, c in enumerate(allc)}
        N = len(allc)
        import scipy.sparse as sp
        coo = A.tocoo()
        A = sp.csr_matrix((coo.data, (coo.row, [gpos[cm_local[c]] for c in coo.col])),
                          shape=(A.shape[0], N))
        self.row_map, self.col_ids = rm, allc
        K = min(self.k + self.oversample, N)
        rng = np.random.default_rng(self.seed)       # same H on every worker
        H = rng.uniform(-1, 1, (N, K))
        W = np.zeros((A.shape[0], K))
        for _ in range(self.iters):
            W = (A @ H) @ np.linalg.pinv(H.T @ H)
            WtW = self._reduce("WtW", W.T @ W)
            AtW = self._reduce("AtW", A.T @ W)
            H = AtW @ np.linalg.pinv(WtW)
        W = (A @ H) @ np.linalg.pinv(H.T @ H)
        # Cholesky-QR (M^T M = L L^T, Q = M L^-T, R = L^T); when the oversampled factors are
        # rank deficient the Gram matrix is only semi-definite and its eigen-decomposition
        # gives the same orthonormal basis restricted to the numerical range
        Tw, Rw = self._orth(self._reduce("WtW", W.T @ W))
        Th, Rh = self._orth(H.T @ H)
        Qw, Qh = W @ Tw, H @ Th
        Ur, S, Vrt = np.linalg.svd(Rw @ Rh.T)
        kk = min(self.k, S.size)
        self.sigma = S[:kk]
        self.U = (Qw @ Ur)[:, :kk]
        self.V = (Qh @ Vrt.T)[:, :kk]

    @staticmethod
    def _orth(G: np.ndarray):
        """(T, R) with Q = M T orthonormal and M = Q R, from the Gram matrix G = M^T M."""
        try:
            L = np.linalg.cholesky(G)
            if np.min(np.abs(np.diag(L))) > 1e-7 * np.max(np.abs(np.diag(L))):
                return np.linalg.inv(L).T, L.T
        except np.linalg.LinAlgError:
            pass
        lam, V = np.linalg.eigh(G)
        keep = lam > 1e-12 * lam.max()
        lam, V = lam[keep], V[:, keep]
        return V / np.sqrt(lam)[None, :], (V * np.sqrt(lam)[None, :]).T

    def dump_result(self):
        if self.get_worker_id() == 0:
            self.paracel_dump_vector(self.sigma.tolist(), "SIGMA_")
            self.paracel_dump_dict({self.col_ids[j]: self.V[j].tolist() for j in range(self.V.shape[0])},
                                   "V_")
        self.paracel_dump_dict({self.row_map[i]: self.U[i].tolist() for i in range(self.U.shape[0])},
                               "U_")
