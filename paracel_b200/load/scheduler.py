"""Load scheduling, hash placement of parsed triples, exchange and id compaction
(reference: include/load/scheduler.hpp:36-343, src/scheduler.cpp:25-113)."""
from __future__ import annotations

from typing import Callable, Hashable, List, Sequence, Tuple

import numpy as np

from .._core import core
from ..parallel.comm import Comm
from ..utils.decomp import npfact2d, npfactx, npfacty
from ..utils.ext import str_split
from ..utils.types import BLK_SZ
from .partition import partition

Triple = Tuple[Hashable, Hashable, float]


def _hash(x) -> int:
    c = core()
    if isinstance(x, (int, np.integer)):
        return c.hash_u64(int(x) & 0xFFFFFFFFFFFFFFFF)
    return c.hash_string(str(x))


class scheduler:
    leader = 0

    def __init__(self, comm: Comm, pattern: str = "fmap", mix: bool = False):
        self.m_comm = comm
        self.pattern = pattern
        self.mix = mix
        self.dim_init()

    def dim_init(self) -> None:
        np_ = self.m_comm.get_size()
        self.npx, self.npy = npfactx(np_)
        if self.pattern == "fsmap":
            self.npx, self.npy = npfact2d(np_)
        if self.pattern == "smap":
            self.npx, self.npy = npfacty(np_)

    def _blk_sz(self) -> int:
        return 1 if self.pattern in ("fvec", "linesplit") else BLK_SZ

    # ---------------------------------------------------------------- loading
    def structure_load(self, part: partition) -> List[str]:
        """Static assignment: rank r reads blocks [r*blk_sz, (r+1)*blk_sz)."""
        b = self._blk_sz()
        r = self.m_comm.get_rank()
        return part.native().load_blocks(r * b, (r + 1) * b)

    def structure_load_handle(self, part: partition, func: Callable[[str], None]) -> None:
        for line in self.structure_load(part):
            func(line)

    def schedule_load(self, part: partition) -> List[str]:
        """Dynamic assignment: the leader reads the first blk_sz blocks, then serves block
        numbers to whichever worker asks next (src/scheduler.cpp:36-95)."""
        comm = self.m_comm
        rk, sz = comm.get_rank(), comm.get_size()
        b = self._blk_sz()
        ntasks = sz * b
        result: List[str] = []
        nat = part.native()
        if sz == 1:
            return nat.load_blocks(0, ntasks)
        if rk == self.leader:
            result.extend(nat.load_blocks(0, b))
            nxt = b
            finished = 0
            # every worker asks until it is told there is nothing left
            while finished < sz - 1:
                src = self._recv_any()
                if nxt < ntasks:
                    comm.send(nxt, src, tag=2015)
                    nxt += 1
                else:
                    comm.send(-1, src, tag=2015)
                    finished += 1
        else:
            while True:
                comm.send(rk, self.leader, tag=2016)
                task = comm.recv(self.leader, tag=2015)
                if task < 0:
                    break
                result.extend(nat.load_blocks(task, task + 1))
        return result

    def _recv_any(self) -> int:
        """Receive a request from any worker (polling the non-leader ranks round robin)."""
        import torch
        import torch.distributed as dist
        comm = self.m_comm
        # gloo supports recv from any source with src=None
        n = torch.zeros(1, dtype=torch.int64)
        src = dist.recv(n, src=None, group=comm.group, tag=2016)
        t = torch.empty(int(n.item()), dtype=torch.uint8)
        dist.recv(t, src=src, group=comm.group, tag=2016)
        import pickle
        who = pickle.loads(t.numpy().tobytes())
        return int(who)

    # ------------------------------------------------------------- placement
    def h(self, i, j, nx: int = None, ny: int = None) -> int:
        nx = self.npx if nx is None else nx
        ny = self.npy if ny is None else ny
        return (_hash(i) % nx) * ny + _hash(j) % ny

    def select(self, i, j=None) -> int:
        if j is None:
            return _hash(i) % self.npx
        return (_hash(i) % self.npx) * self.npy + _hash(j) % self.npy

    def lines_organize(self, lines: Sequence[str], parser_func: Callable[[str], List[str]],
                       numeric: bool = True) -> List[List[Triple]]:
        """Parse lines into (a, b, w) triples and bin them by destination rank.  Accepted
        shapes: ``a b`` / ``a b:0.2``; with ``mix`` an adjacency list ``a b c`` or
        ``a b|0.2 c|0.4``; otherwise exactly ``a b w``."""
        slots: List[List[Triple]] = [[] for _ in range(self.m_comm.get_size())]
        cvt = (lambda s: int(s)) if numeric else (lambda s: s)

        def item(a, it):
            tmp = str_split(it, ":| ")
            b = cvt(tmp[0])
            w = float(tmp[1]) if len(tmp) > 1 else 1.0
            slots[self.h(a, b)].append((a, b, w))

        for line in lines:
            if not line:
                continue
            stf = parser_func(line)
            if len(stf) < 2:
                continue
            a = cvt(stf[0])
            if len(stf) == 2:
                item(a, stf[1])
            elif self.mix:
                for it in stf[1:]:
                    item(a, it)
            else:
                if len(stf) != 3:
                    raise ValueError(f"lines_organize: unsupported line format: {line!r}")
                b = cvt(stf[1])
                slots[self.h(a, b)].append((a, b, float(stf[2])))
        return slots

    def exchange(self, slots: List[List[Triple]]) -> List[Triple]:
        """All-to-all of the per-destination bins; returns the triples this rank owns."""
        got = self.m_comm.alltoall(slots)
        out: List[Triple] = []
        for part in got:
            out.extend(part)
        return out

    def index_mapping(self, triples: Sequence[Triple]):
        """Dense renumbering of row and column ids.  Ranks in the same grid row share the
        row ids, ranks in the same grid column share the column ids (union by ring
        broadcast over the row / column sub-communicators).  Returns
        (renumbered triples, rm: index -> row id, cm: index -> column id)."""
        rk = self.m_comm.get_rank()
        rowcolor, colcolor = rk // self.npy, rk % self.npy
        col_comm = self.m_comm.split(colcolor)
        row_comm = self.m_comm.split(rowcolor)
        rows = sorted({t[0] for t in triples}, key=_sort_key)
        cols = sorted({t[1] for t in triples}, key=_sort_key)
        new_rows, new_cols = set(), set()
        row_comm.bcastring(rows, lambda tmp: new_rows.update(tmp))
        col_comm.bcastring(cols, lambda tmp: new_cols.update(tmp))
        rm = {i: r for i, r in enumerate(sorted(new_rows, key=_sort_key))}
        cm = {i: c for i, c in enumerate(sorted(new_cols, key=_sort_key))}
        rev_rm = {r: i for i, r in rm.items()}
        rev_cm = {c: i for i, c in cm.items()}
        stf = [(rev_rm[a], rev_cm[b], w) for a, b, w in triples]
        return stf, rm, cm


def _sort_key(x):
    return (0, x) if isinstance(x, (int, np.integer)) else (1, str(x))
