"""Decision-tree recommender builder (reference:
alg/recommendation/decision_tree_rec/decision_tree_builder.hpp:40-360).

For every tree index k in [tree_start_index, tree_end_index] a binary tree with
``2^level - 1`` nodes is grown breadth first.  A node holds an item; users whose factor has
a non-negative inner product with the item's factor go to the "like" child, the others to
the "hate" child.  Each worker scores its shard of the items by the summed squared distance
of the users to their side's mean factor (splits more lopsided than 3:1 are skipped); the
global minimum is found with the min-pair handler.  The root of tree k takes the k-th
smallest error instead (via write_multi + read_special + remove), which makes the trees
differ.  Output: ``tree_0`` and ``average_user_factor_<k>``."""
from __future__ import annotations

import os
from collections import deque
from typing import Dict, List

import numpy as np

from ..paralg import paralg
from ..utils.dump import to_string
from ..utils.ext import str_split, todir

SENTINEL_ITEM = 2 ** 63 - 1


class decision_tree_builder_factor(paralg):
    def __init__(self, comm, hosts_dct_str, user_fac_input: str, item_fac_input: str,
                 output: str = "", handle_file: str = "", level: int = 3, tree_start_index: int = 0,
                 tree_end_index: int = 0, **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.uinput, self.iinput, self.handle_file = user_fac_input, item_fac_input, handle_file
        self.level, self.N_start, self.N_end = int(level), int(tree_start_index), int(tree_end_index)
        self.trees: Dict[int, List[int]] = {k: [] for k in range(self.N_start, self.N_end + 1)}
        self.avg_ufacs: Dict[int, List[List[float]]] = {k: [] for k in range(self.N_start, self.N_end + 1)}

    @staticmethod
    def _parse(lines):
        ids, rows = [], []
        for line in lines:
            if not line:
                continue
            t = str_split(line, "\t")
            ids.append(int(t[0]))
            rows.append([float(x) for x in str_split(t[1], "|")])
        return ids, np.asarray(rows, dtype=np.float64)

    def solve(self):
        _, self.ufac = self._parse(self.paracel_loadall(self.uinput))
        self.kdim = self.ufac.shape[1]
        self.item_ids, self.ifac = self._parse(self.paracel_load(self.iinput))
        if self.item_ids:
            self.paracel_write_multi({f"ifac_{i}": f.tolist() for i, f in zip(self.item_ids, self.ifac)})
        users = np.arange(self.ufac.shape[0])
        if self.get_worker_id() == 0:
            for n in range(self.N_start, self.N_end + 1):
                self.avg_ufacs[n].append(self.cal_avg_pu(users))
        self.paracel_sync()
        for k in range(self.N_start, self.N_end + 1):
            self.build(k, users)
            self.paracel_sync()

    def cal_avg_pu(self, uset) -> List[float]:
        if len(uset) == 0:
            return [0.0] * self.kdim
        return self.ufac[uset].mean(0).tolist()

    def _scores(self, U, occur) -> Dict[int, float]:
        out: Dict[int, float] = {}
        if len(U) == 0 or len(self.item_ids) == 0:
            return out
        P = self.ufac[U]
        like = (P @ self.ifac.T) >= 0.0             # users x items
        nl = like.sum(0)
        nh = len(U) - nl
        for j, iid in enumerate(self.item_ids):
            if iid in occur or nl[j] == 0 or nh[j] == 0:
                continue
            if nl[j] // nh[j] >= 3 or nh[j] // nl[j] >= 3:
                continue
            L, Hh = P[like[:, j]], P[~like[:, j]]
            out[iid] = float(((L - L.mean(0)) ** 2).sum() + ((Hh - Hh.mean(0)) ** 2).sum())
        return out

    def find_node(self, tree_indx, U, occur, Q, is_root) -> int:
        if len(U) == 0:
            Q.append(np.zeros(0, dtype=np.int64))
            Q.append(np.zeros(0, dtype=np.int64))
            return SENTINEL_ITEM
        err = self._scores(U, occur)
        partition_id = SENTINEL_ITEM
        if is_root:
            best = sorted(err.items(), key=lambda kv: kv[1])[: tree_indx + 1]
            tmp = {f"err_{i}": e for i, e in best}
            if tmp:
                self.paracel_write_multi(tmp)
            self.paracel_sync()
            cand = sorted(self.paracel_read_special("", "prefix:err_").items(), key=lambda kv: kv[1])
            if cand:
                partition_id = int(cand[min(tree_indx, len(cand) - 1)][0][4:])
            self.paracel_sync()
            for k in tmp:
                self.paracel_remove(k)
            self.paracel_sync()
        else:
            mine = min(err.items(), key=lambda kv: kv[1]) if err else (SENTINEL_ITEM, float("inf"))
            self.paracel_sync()
            self.paracel_bupdate("smallest_error", [mine[0], mine[1]], self.handle_file,
                                 "smallest_error_updater")
            self.paracel_sync()
            partition_id = int(self.paracel_read("smallest_error")[0])
            self.paracel_sync()
            if self.get_worker_id() == 0:
                self.paracel_remove("smallest_error")
            self.paracel_sync()
        if partition_id == SENTINEL_ITEM:
            Q.append(np.zeros(0, dtype=np.int64))
            Q.append(np.zeros(0, dtype=np.int64))
            return partition_id
        p_i = np.asarray(self.paracel_read(f"ifac_{partition_id}"))
        like = (self.ufac[U] @ p_i) >= 0.0
        Ul, Uh = U[like], U[~like]
        if self.get_worker_id() == 0:
            self.avg_ufacs[tree_indx].append(self.cal_avg_pu(Ul))
            self.avg_ufacs[tree_indx].append(self.cal_avg_pu(Uh))
        Q.append(Ul)
        Q.append(Uh)
        return partition_id

    def build(self, tree_indx, users):
        Q = deque([users])
        occur = set()
        cnt, total = 0, (1 << self.level) - 1
        while Q and cnt < total:
            UU = Q.popleft()
            pid = self.find_node(tree_indx, UU, occur, Q, is_root=(cnt == 0))
            occur.add(pid)
            self.trees[tree_indx].append(pid)
            cnt += 1

    def dump(self):
        if self.get_worker_id() != 0:
            return
        os.makedirs(self.output or ".", exist_ok=True)
        with open(todir(self.output) + "tree_0", "w") as f:
            for k in range(self.N_start, self.N_end + 1):
                f.write(f"tree_{k}\t" + "|".join(str(x) for x in self.trees[k]) + "\n")
        nodes = (1 << self.level) - 1
        for k in range(self.N_start, self.N_end + 1):
            with open(todir(self.output) + f"average_user_factor_{k}", "w") as f:
                for row in self.avg_ufacs[k][:nodes]:
                    f.write("|".join(to_string(float(x)) for x in row) + "\n")

    dump_result = dump
