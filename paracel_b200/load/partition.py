"""Byte-range partition of a multi-file corpus (reference:
include/load/partition.hpp:30-241; native implementation in csrc/core/textio.hpp)."""
from __future__ import annotations

from typing import Callable, List, Sequence

from .._core import core
from ..utils.types import BLK_SZ


class partition:
    def __init__(self, namelst: Sequence[str], np_: int, pattern: str = "linesplit"):
        self.namelst = list(namelst)
        self.np = int(np_)
        self.pattern = pattern
        self._p = None

    def files_partition(self, blk_sz: int = BLK_SZ) -> None:
        if self.pattern in ("linesplit", "fvec"):
            blk_sz = 1
        self.blk_sz = blk_sz
        self._p = core().FilePartition(self.namelst, self.np, blk_sz)

    def file_partition(self, fname: str):
        """Single-file form used by the reference's partition test."""
        p = core().FilePartition([fname], self.np, 1)
        return list(p.starts), list(p.ends)

    def get_start_list(self) -> List[int]:
        return list(self._p.starts)

    def get_end_list(self) -> List[int]:
        return list(self._p.ends)

    def files_load_lines_impl(self, st: int, en: int, func: Callable[[str], None] = None):
        lines = self._p.load_lines(st, en)
        if func is None:
            return lines
        for l in lines:
            func(l)

    def file_load_lines_impl(self, fname: str, st: int, en: int) -> List[str]:
        return core().FilePartition([fname], 1, 1).load_lines(st, en)

    def native(self):
        return self._p
