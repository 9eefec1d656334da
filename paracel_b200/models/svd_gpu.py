"""Truncated SVD on GPUs (device path of alg/recommendation/svd/svd.hpp:40-310 and of the
complete serial version tool/svd_serial.cpp:40-190).

``SvdGpu`` is a ``paralg`` subclass on the device backend.  The sparse matrix A is
row-partitioned over the ranks (CSR in HBM), H (N x K) is replicated, W (local rows x K) is
local.  Stage 1 repeats ``W = A H (H^T H)^-1``, ``H = A^T W (W^T W)^-1``; the K x K Gram matrix
``W^T W`` and the N x K product ``A^T W`` are summed over the ranks THROUGH the parameter
tables, as the reference does with its ``WtW`` / ``AtW_<k>`` keys (svd.hpp:137-181): each rank
writes its part into ``paracel_delta_buffer(key)`` and a collective ``paracel_bupdate`` with the
``svd_updater`` (add) handler reduces them into the owners' shards, ``paracel_read`` gathers the
sum.  Stage 2 is the Cholesky-QR of W and H (``M^T M = R^T R``, ``Q = M R^-1``) and the SVD of the
K x K matrix ``R_W R_H^T`` (on the host, svd.hpp:294-298), ``U = Q_W U_r``, ``V = Q_H V_r``.

Kernels: CSR products ``A.H`` / ``A^T.W`` and the small Cholesky factor (csrc/cuda/svd.cu), the
Gram matrix (``pcl_gram``), and the tcgen05 GEMM (3xTF32) for the skinny products with K x K
matrices."""
from __future__ import annotations

import os

import torch

from ..ops.gemm import gemm_nt
from ..ops.misc import gram
from ..ops.svd import chol_factor, spmm_csr, spmm_csr_t
from ..paralg import paralg


def _orth_fallback(G: torch.Tensor):
    """(T, R) from the eigen-decomposition of a semi-definite Gram matrix restricted to its
    numerical range: Q = M T is orthonormal and M = Q R."""
    lam, V = torch.linalg.eigh(G.double().cpu())
    keep = lam > 1e-12 * lam.max()
    lam, V = lam[keep], V[:, keep]
    T = (V / lam.sqrt()[None, :]).float()
    R = (V * lam.sqrt()[None, :]).T.float()
    return T.to(G.device), R.to(G.device)


class SvdGpu(paralg):
    def __init__(self, n_cols: int, k: int = 2, iters: int = 20, oversample: int = 10, seed: int = 0,
                 group=None, device=None, comm=None, hosts_dct_str=None, output: str = "",
                 update_function: str = "svd_updater"):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.world, self.rank, self.group = self.get_worker_size(), self.get_worker_id(), group
        self.N, self.k, self.iters, self.seed = int(n_cols), int(k), int(iters), seed
        K = min(self.k + int(oversample), self.N)
        self.K = min((K + 3) // 4 * 4, 112)
        self.update_function = update_function
        self.paracel_dense_table("WtW", self.K * self.K, handler=update_function)
        self.paracel_dense_table("AtW", self.N * self.K, handler=update_function)

    def load(self, row_ptr: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor):
        """This rank's rows of A as CSR (int64 row_ptr, int32 global column ids, fp32 values)."""
        from ..ops import _lib
        dev = self.device
        self.row_ptr = row_ptr.to(dev, torch.int64).contiguous()
        self.cols = cols.to(dev, torch.int32).contiguous()
        self.vals = vals.to(dev, torch.float32).contiguous()
        _lib.validate_ids(self.cols, 0, self.N, "SVD input (column ids)")
        self.m = self.row_ptr.numel() - 1

    def _reduce(self, key: str, part: torch.Tensor) -> torch.Tensor:
        """Sum of ``part`` over the ranks through the table ``key``: owners start from zero, a
        collective bupdate adds every rank's part, a read gathers the result."""
        self.paracel_local_shard(key).zero_()
        buf = self.paracel_delta_buffer(key)
        buf.copy_(part.reshape(-1))
        self.paracel_bupdate(key, buf, "", self.update_function, collective=True)
        return self.paracel_read(key).view(part.shape).clone()

    def _times_inverse(self, M: torch.Tensor, G: torch.Tensor) -> torch.Tensor:
        """``M @ pinv(G)`` for a K x K Gram matrix: ``(M T) T^T`` with the Cholesky factor, or
        the pseudo-inverse when G is rank deficient (the oversampled factors can be)."""
        if M.shape[0] == 0:
            return M
        T, _, info = chol_factor(G)
        if info != 0:
            Tf, _ = _orth_fallback(G)
            return (M @ Tf) @ Tf.T
        return gemm_nt(gemm_nt(M, T.T.contiguous(), precise=True), T, precise=True)

    def _orth(self, G: torch.Tensor):
        T, R, info = chol_factor(G, rel_tol=1e-7)
        if info != 0:
            return _orth_fallback(G)
        return T, R

    def solve(self):
        dev, K, N = self.device, self.K, self.N
        g = torch.Generator()
        g.manual_seed(self.seed)
        H = (torch.rand(N, K, generator=g) * 2 - 1).to(dev)      # same H on every rank
        A = (self.row_ptr, self.cols, self.vals)
        for _ in range(self.iters):
            W = self._times_inverse(spmm_csr(*A, H), gram(H))
            WtW = self._reduce("WtW", gram(W) if self.m else torch.zeros(K, K, device=dev))
            AtW = self._reduce("AtW", spmm_csr_t(*A, W, torch.zeros(N, K, device=dev)))
            H = self._times_inverse(AtW, WtW)
        W = self._times_inverse(spmm_csr(*A, H), gram(H))
        Tw, Rw = self._orth(self._reduce("WtW", gram(W) if self.m else torch.zeros(K, K, device=dev)))
        Th, Rh = self._orth(gram(H))
        def times(M, T):      # M @ T on the tensor cores when T is square
            if M.shape[0] == 0 or T.shape[0] != T.shape[1]:
                return M @ T
            return gemm_nt(M, T.T.contiguous(), precise=True)
        Qw, Qh = times(W, Tw), times(H, Th)
        Ur, S, Vrt = torch.linalg.svd((Rw @ Rh.T).double().cpu())      # small K x K problem on the host
        kk = min(self.k, S.numel())
        self.sigma = S[:kk].clone()
        self.U = (Qw @ Ur.float().to(dev))[:, :kk].contiguous()
        self.V = (Qh @ Vrt.T.float().to(dev))[:, :kk].contiguous()
        self.paracel_sync()
        self.paracel_check()

    def dump_result(self, outdir: str = "", row_names=None, col_names=None):
        """SIGMA_0 and V_0 from worker 0, U_<rank> from every worker (tool/svd_serial.cpp:140-153)."""
        from ..utils.dump import dump_dict_vector, dump_vector
        outdir = outdir or self.output
        os.makedirs(outdir, exist_ok=True)
        if self.rank == 0:
            dump_vector(self.sigma.tolist(), os.path.join(outdir, "SIGMA_0"))
            cn = col_names if col_names is not None else list(range(self.N))
            dump_dict_vector({cn[j]: row for j, row in enumerate(self.V.cpu().tolist())},
                             os.path.join(outdir, "V_0"))
        rn = row_names if row_names is not None else list(range(self.m))
        dump_dict_vector({rn[j]: row for j, row in enumerate(self.U.cpu().tolist())},
                         os.path.join(outdir, f"U_{self.rank}"))
        self.paracel_sync()

    def free(self):
        self.close()
