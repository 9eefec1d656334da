"""k-means (reference: alg/clustering/kmeans/kmeans.hpp:40-200).

Host path (paralg): input ``id\\tf1,f2,...`` rows (``fvec``); worker 0 seeds the centres
with its first k rows under key ``clusters_-1``; each round reads ``clusters_{rd-1}``,
assigns every local row to its nearest centre, all-reduces the cluster counts, pushes
``local_sum / global_count`` with the add handler under ``clusters_{rd}``; finally the
groups are merged through ``kmeans_result``.

Device path (``kmeans_gpu``): centres are a ``DenseReadGemm`` parameter (range-sharded
over the ranks), the assignment is the tcgen05 GEMM with the fused arg-min epilogue (and the
all-gather of the centres fused in), per-cluster sums are accumulated with index_add and
pushed through a ``DenseTable`` with the add handler."""
from __future__ import annotations

from typing import Dict, List

import numpy as np

from ..paralg import paralg
from ..utils.ext import str_split


def _fvec_parser(line: str) -> List[str]:
    r = str_split(line, "\t")
    return [r[0]] + str_split(r[1], ",")


class kmeans(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", dtype: str = "fvec",
                 kclusters: int = 2, update_file: str = "", update_funcs=None, rounds: int = 1, **kw):
        super().__init__(hosts_dct_str, comm, output, rounds, **kw)
        self.input, self.dtype, self.kclusters = input, dtype, int(kclusters)
        self.update_file = update_file
        self.update_funcs = list(update_funcs or ["local_update_kmeans_clusters",
                                                  "local_update_kmeans_groups"])
        self.clusters: List[List[float]] = []
        self.groups: Dict[int, List[str]] = {}

    def init(self):
        if self.dtype != "fvec":
            raise NotImplementedError("only dense 'fvec' input is supported (as in the reference)")
        self.blk_dmtx, self.row_map = self.paracel_load_as_matrix(
            self.input, _fvec_parser, pattern="fvec", numeric=False)
        if self.get_worker_id() == 0:
            init_clusters = [self.blk_dmtx[i].tolist() for i in range(self.kclusters)]
            self.paracel_write("clusters_-1", init_clusters)
        self.paracel_sync()

    def assign(self, C: np.ndarray) -> np.ndarray:
        X = self.blk_dmtx
        d2 = (C * C).sum(1)[None, :] - 2.0 * X @ C.T
        return np.argmin(d2, axis=1)

    def learning(self):
        self.paracel_register_bupdate(self.update_file, self.update_funcs[0])
        owner = np.zeros(0, dtype=np.int64)
        k, X = self.kclusters, self.blk_dmtx
        for rd in range(self.rounds):
            C = np.asarray(self.paracel_read(f"clusters_{rd - 1}"), dtype=np.float64)
            owner = self.assign(C) if X.shape[0] else np.zeros(0, dtype=np.int64)
            cnt = np.bincount(owner, minlength=k).astype(np.int64)
            sums = np.zeros((k, C.shape[1]))
            np.add.at(sums, owner, X)
            cnt_global = np.asarray(self.get_comm().allreduce(cnt.tolist()), dtype=np.float64)
            part = sums / np.maximum(cnt_global, 1.0)[:, None]
            self.paracel_bupdate(f"clusters_{rd}", part.tolist())
            self.paracel_sync()
        self.clusters = self.paracel_read(f"clusters_{self.rounds - 1}")
        groups: Dict[int, List[str]] = {}
        for i, c in enumerate(owner.tolist()):
            groups.setdefault(int(c), []).append(str(self.row_map[i]))
        self.paracel_bupdate("kmeans_result", groups, self.update_file, self.update_funcs[1])
        self.paracel_sync()
        self.groups = {int(k_): v for k_, v in self.paracel_read("kmeans_result").items()}

    def solve(self):
        self.init()
        self.paracel_sync()
        self.learning()

    def dump_result(self):
        if self.get_worker_id() == 0:
            self.paracel_dump_dict(self.groups, "kmeans_")
            self.paracel_dump_dict({i: c for i, c in enumerate(self.clusters)}, "centers_")
