"""Distributed loader: lines -> partitioned graphs and matrices (reference:
include/load/loader.hpp:50-394)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Sequence, Union

import numpy as np

from ..graph import bigraph_continuous
from ..parallel.comm import Comm
from ..utils.ext import expand
from .parser import parser_a
from .partition import partition
from .scheduler import scheduler


class loader:
    def __init__(self, filenames: Union[str, Sequence[str]], comm: Comm,
                 parser: Callable[[str], List[str]] = parser_a, pattern: str = "fmap",
                 mix: bool = False):
        self.filenames = filenames
        self.m_comm = comm
        self.parserfunc = parser
        self.pattern = pattern
        self.mix = mix or pattern == "fset"  # fset lines are adjacency sets: a b:0.2|c:0.4

    def _partition(self) -> partition:
        names = expand(self.filenames)
        if not names:
            raise FileNotFoundError(f"no input file matches {self.filenames!r}")
        p = partition(names, self.m_comm.get_size(), self.pattern)
        p.files_partition()
        return p

    def load(self) -> List[str]:
        """Dynamic (leader-scheduled) load of this rank's share of the lines."""
        sch = scheduler(self.m_comm, self.pattern, self.mix)
        lines = sch.schedule_load(self._partition())
        self.m_comm.synchronize()
        return lines

    def fixload(self) -> List[str]:
        """Static load: rank r reads its fixed block range."""
        sch = scheduler(self.m_comm, self.pattern, self.mix)
        lines = sch.structure_load(self._partition())
        self.m_comm.synchronize()
        return lines

    def fixload_handle(self, func: Callable[[str], None]) -> None:
        sch = scheduler(self.m_comm, self.pattern, self.mix)
        sch.structure_load_handle(self._partition(), func)

    # ------------------------------------------------------------- builders
    def _owned_triples(self, lines: Sequence[str], numeric: bool):
        sch = scheduler(self.m_comm, self.pattern, self.mix)
        slots = sch.lines_organize(lines, self.parserfunc, numeric=numeric)
        self.m_comm.synchronize()
        stf = sch.exchange(slots)
        self.m_comm.synchronize()
        return sch, stf

    def create_graph(self, lines: Sequence[str], grp, numeric: bool = True):
        """Fill ``grp`` (digraph / bigraph / undirected_graph) with the edges this rank owns
        under the load pattern.  For ``bigraph_continuous`` returns (rm, cm) id maps."""
        sch, stf = self._owned_triples(lines, numeric)
        if isinstance(grp, bigraph_continuous):
            stf_new, rm, cm = sch.index_mapping(stf)
            self.m_comm.synchronize()
            grp.resize(len(rm))
            for a, b, w in stf_new:
                grp.add_edge(a, b, w)
            return rm, cm
        for a, b, w in stf:
            grp.add_edge(a, b, w)
        return None

    def create_matrix(self, lines: Sequence[str], dense: bool = False, numeric: bool = True):
        """Sparse case: returns (csr block, rm, cm) with dense local numbering of the rows
        and columns present on this rank's grid row / column.  Dense (``fvec``) case:
        lines are ``id<sep>f1<sep>...`` and the result is (ndarray, rm)."""
        if dense:
            rm: Dict[int, Any] = {}
            rows = []
            for indx, line in enumerate(l for l in lines if l):
                stf = self.parserfunc(line)
                rm[indx] = int(stf[0]) if numeric else stf[0]
                rows.append([float(x) for x in stf[1:]])
            mtx = np.asarray(rows, dtype=np.float64) if rows else np.zeros((0, 0))
            return mtx, rm
        import scipy.sparse as sp
        sch, stf = self._owned_triples(lines, numeric)
        stf_new, rm, cm = sch.index_mapping(stf)
        self.m_comm.synchronize()
        if stf_new:
            r, c, v = zip(*stf_new)
        else:
            r, c, v = (), (), ()
        blk = sp.csr_matrix((np.asarray(v, dtype=np.float64),
                             (np.asarray(r, dtype=np.int64), np.asarray(c, dtype=np.int64))),
                            shape=(len(rm), len(cm)))
        return blk, rm, cm
