"""Matrix factorisation by SGD on the host parameter server (reference:
alg/recommendation/matrix_factorization/mf.hpp:46-500, mf_driver.cpp).

Keys: ``W_<uid>`` / ``H_<iid>`` (factor rows), ``usr_bias_<uid>`` / ``item_bias_<iid>``,
``<uid>_u_cnt`` / ``<iid>_i_cnt`` (how many workers hold the row; the push weight is its
inverse).  Input ``user item date rating`` (space separated, the date is dropped), loaded
with the ``fsmap`` 2-D pattern.  SSP is on by default (``limit_s = 3``) as in the reference.
The GPU version of the same round structure is ``paracel_b200.models.mf_gpu.MfSgdGpu``."""
from __future__ import annotations

import math
from typing import List, Tuple

import numpy as np

from .._core import core
from ..graph import bigraph
from ..paralg import paralg
from ..utils.ext import str_split


def _mf_parser(line: str) -> List[str]:
    lst = str_split(line, " ")
    if len(lst) >= 4:
        del lst[2]
    return lst


class matrix_factorization(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, predict_input: str = "", output: str = "",
                 update_file: str = "", update_funcs=None, filter_file: str = "", filter_funcs=None,
                 k: int = 80, rounds: int = 1, alpha: float = 0.005, beta: float = 0.01,
                 debug: bool = False, ssp_switch: bool = True, limit_s: int = 3, seed: int = 0, **kw):
        super().__init__(hosts_dct_str, comm, output, rounds, limit_s, ssp_switch, **kw)
        self.input, self.predict_input = input, predict_input
        self.update_file = update_file
        self.update_funcs = list(update_funcs or ["cnt_updater", "mf_fac_updater", "mf_bias_updater"])
        self.filter_file = filter_file
        self.filter_funcs = list(filter_funcs or ["mf_ubias_filter", "mf_ibias_filter", "mf_W_filter",
                                                  "mf_H_filter"])
        self.fac_dim, self.alpha, self.beta, self.debug = int(k), float(alpha), float(beta), debug
        self.rng = np.random.default_rng(seed + 7919 * self.worker_comm.get_rank())
        self.miu = 0.0
        self.loss_error_train: List[float] = []
        self.predv: List[Tuple[int, int, float]] = []

    # -------------------------------------------------------------- set-up
    def init_parameters(self):
        self.rating_graph = bigraph()
        self.paracel_load_as_graph(self.rating_graph, self.input, _mf_parser, "fsmap")
        u, i, r = self.rating_graph.to_coo()
        self.rating_sz = int(u.size)
        self.users = np.unique(u)
        self.items = np.unique(i)
        self.ru = np.searchsorted(self.users, u).astype(np.int64)
        self.ri = np.searchsorted(self.items, i).astype(np.int64)
        self.rr = np.ascontiguousarray(r, dtype=np.float64)
        self.paracel_sync()
        tot = self.worker_comm.allreduce([float(r.sum()), float(self.rating_sz)])
        self.miu = tot[0] / max(tot[1], 1.0)
        self.total_sz = int(tot[1])
        k = self.fac_dim
        nU, nI = self.users.size, self.items.size
        self.W = 0.1 * self.rng.random((nU, k))
        self.H = 0.1 * self.rng.random((nI, k))
        self.ub = 0.1 * self.rng.random(nU)
        self.ib = 0.1 * self.rng.random(nI)
        ukeys = [str(x) for x in self.users.tolist()]
        ikeys = [str(x) for x in self.items.tolist()]
        self.paracel_bupdate_multi([x + "_u_cnt" for x in ukeys], [1] * nU, self.update_file,
                                   self.update_funcs[0])
        self.paracel_write_multi({"W_" + x: self.W[j].tolist() for j, x in enumerate(ukeys)})
        self.paracel_write_multi({"usr_bias_" + x: float(self.ub[j]) for j, x in enumerate(ukeys)})
        self.paracel_bupdate_multi([x + "_i_cnt" for x in ikeys], [1] * nI, self.update_file,
                                   self.update_funcs[0])
        self.paracel_write_multi({"H_" + x: self.H[j].tolist() for j, x in enumerate(ikeys)})
        self.paracel_write_multi({"item_bias_" + x: float(self.ib[j]) for j, x in enumerate(ikeys)})
        self.paracel_sync()
        cx = self.paracel_read_multi([x + "_u_cnt" for x in ukeys]) if nU else []
        cy = self.paracel_read_multi([x + "_i_cnt" for x in ikeys]) if nI else []
        self.wgtx = 1.0 / np.maximum(np.asarray(cx, dtype=np.float64), 1.0)
        self.wgty = 1.0 / np.maximum(np.asarray(cy, dtype=np.float64), 1.0)
        self.ukeys, self.ikeys = ukeys, ikeys
        self.paracel_sync()

    # --------------------------------------------------------------- rounds
    def read_mf_paras(self):
        if self.ukeys:
            self.W = np.asarray(self.paracel_read_multi(["W_" + x for x in self.ukeys]), dtype=np.float64)
            self.ub = np.asarray(self.paracel_read_multi(["usr_bias_" + x for x in self.ukeys]),
                                 dtype=np.float64)
        if self.ikeys:
            self.H = np.asarray(self.paracel_read_multi(["H_" + x for x in self.ikeys]), dtype=np.float64)
            self.ib = np.asarray(self.paracel_read_multi(["item_bias_" + x for x in self.ikeys]),
                                 dtype=np.float64)
        self.W, self.H = np.ascontiguousarray(self.W), np.ascontiguousarray(self.H)
        self.ub, self.ib = np.ascontiguousarray(self.ub), np.ascontiguousarray(self.ib)

    def estimate(self, ju: int, ji: int) -> float:
        p = self.miu + self.ub[ju] + self.ib[ji] + float(self.W[ju] @ self.H[ji])
        return min(5.0, max(1.0, p))

    def cal_rmse(self) -> float:
        if self.rating_sz:
            p = self.miu + self.ub[self.ru] + self.ib[self.ri] + (self.W[self.ru] * self.H[self.ri]).sum(1)
            e = self.rr - np.clip(p, 1.0, 5.0)
            s = float((e * e).sum())
        else:
            s = 0.0
        tot = self.worker_comm.allreduce([s, float(self.rating_sz)])
        return math.sqrt(tot[0] / max(tot[1], 1.0))

    def learning(self):
        for rd in range(self.rounds):
            self.read_mf_paras()
            if self.debug:
                self.loss_error_train.append(self.cal_rmse())
            oW, oH, oub, oib = self.W.copy(), self.H.copy(), self.ub.copy(), self.ib.copy()
            core().mf_sgd_pass(self.ru, self.ri, self.rr, self.W, self.H, self.ub, self.ib, self.miu,
                               self.alpha, self.beta)
            dW = self.wgtx[:, None] * (self.W - oW)
            dH = self.wgty[:, None] * (self.H - oH)
            self.paracel_bupdate_multi(["W_" + x for x in self.ukeys], dW.tolist(), self.update_file,
                                       self.update_funcs[1])
            self.paracel_bupdate_multi(["H_" + x for x in self.ikeys], dH.tolist(), self.update_file,
                                       self.update_funcs[1])
            self.paracel_sync()
            self.paracel_bupdate_multi(["usr_bias_" + x for x in self.ukeys],
                                       (self.wgtx * (self.ub - oub)).tolist(), self.update_file,
                                       self.update_funcs[2])
            self.paracel_bupdate_multi(["item_bias_" + x for x in self.ikeys],
                                       (self.wgty * (self.ib - oib)).tolist(), self.update_file,
                                       self.update_funcs[2])
            self.paracel_sync()
            self.iter_commit()
        self.read_mf_paras()
        if self.debug:
            self.loss_error_train.append(self.cal_rmse())
        self.paracel_sync()

    def solve(self):
        self.init_parameters()
        self.set_total_iters(self.rounds)
        self.paracel_sync()
        self.learning()
        self.paracel_sync()

    def predict(self):
        if not self.predict_input:
            return
        lines = [l for l in self.paracel_load(self.predict_input) if l]
        W = {int(k.rsplit("_", 1)[1]): v for k, v in
             self.paracel_read_special(self.filter_file, self.filter_funcs[2]).items()}
        H = {int(k.rsplit("_", 1)[1]): v for k, v in
             self.paracel_read_special(self.filter_file, self.filter_funcs[3]).items()}
        ub = {int(k.rsplit("_", 1)[1]): v for k, v in
              self.paracel_read_special(self.filter_file, self.filter_funcs[0]).items()}
        ib = {int(k.rsplit("_", 1)[1]): v for k, v in
              self.paracel_read_special(self.filter_file, self.filter_funcs[1]).items()}
        for line in lines:
            a, b = str_split(line, ",")[:2]
            uid, iid = int(a), int(b)
            if uid not in W or iid not in H:
                self.predv.append((uid, iid, self.miu))
            else:
                p = self.miu + ub.get(uid, 0.0) + ib.get(iid, 0.0) + float(np.dot(W[uid], H[iid]))
                self.predv.append((uid, iid, min(5.0, max(1.0, p))))

    def dump_result(self):
        if self.get_worker_id() == 0:
            self.paracel_dump_dict({"miu": self.miu, "rating_sz": float(self.total_sz)}, "miu_")
            tear = lambda s: s.rsplit("_", 1)[1]
            first = {"ubias_": True, "ibias_": True, "W_": True, "H_": True}
            for prefix, fidx in (("ubias_", 0), ("ibias_", 1), ("W_", 2), ("H_", 3)):
                def handler(d, prefix=prefix):
                    self.paracel_dump_dict({tear(k): v for k, v in d.items()}, prefix,
                                           append_flag=not first[prefix])
                    first[prefix] = False
                self.paracel_read_special_handle(self.filter_file, self.filter_funcs[fidx], handler)
            if self.debug:
                self.paracel_dump_vector(self.loss_error_train, "mf_loss_error_train_", "\n")
        self.paracel_dump_vector(self.predv, "pred_v_", "\n")
        self.paracel_sync()
