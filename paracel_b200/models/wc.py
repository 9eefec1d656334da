"""Word count (reference: alg/misc/word_count/wc.hpp:46-190, wc_driver.cpp).

Three variants as in the reference: ``learning_slow_demo`` (one bupdate per word
occurrence), ``learning_slow`` (local combine, one bupdate per distinct word) and
``learning`` (local combine, words hashed into 100 buckets, one dictionary-merge
bupdate per bucket, top-k over the buckets with a min-heap)."""
from __future__ import annotations

import heapq
import re
from collections import Counter
from typing import Dict, List, Tuple

from .._core import core
from ..paralg import paralg

_WORD = re.compile(r"[^-a-zA-Z0-9_]")


class word_count(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", topk: int = 10,
                 handle_file: str = "", update_function: str = "wc_updater",
                 filter_function: str = "wc_filter", **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input, self.topk = input, int(topk)
        self.handle_file = handle_file
        self.update_function, self.filter_function = update_function, filter_function
        self.result: List[Tuple[str, int]] = []

    @staticmethod
    def parser(line: str) -> List[str]:
        return [w for w in _WORD.split(line) if w]

    def _local_counts(self, lines) -> Counter:
        c: Counter = Counter()
        for line in lines:
            c.update(self.parser(line))
        return c

    def learning_slow_demo(self, lines):
        for line in lines:
            for w in self.parser(line):
                self.paracel_bupdate(w, 1, self.handle_file, "wc_updater_slow")
        self.paracel_sync()
        self.result = self.paracel_read_topk(self.topk)

    def learning_slow(self, lines):
        for w, n in self._local_counts(lines).items():
            self.paracel_bupdate(w, n, self.handle_file, "wc_updater_slow")
        self.paracel_sync()
        self.result = self.paracel_read_topk(self.topk)

    def learning(self, lines):
        tmp = self._local_counts(lines)
        dct_sz = 100
        local_vd: List[Dict[str, int]] = [dict() for _ in range(dct_sz)]
        h = core().hash_string
        for w, n in tmp.items():
            local_vd[h(w) % dct_sz][w] = n
        self.paracel_sync()
        for k, d in enumerate(local_vd):
            if d:
                self.paracel_bupdate(f"key_{k}", d, self.handle_file, self.update_function)
        self.paracel_sync()
        heap: List[Tuple[int, str]] = []

        def handler(d):
            for _, bucket in d.items():
                for w, n in bucket.items():
                    if len(heap) < self.topk:
                        heapq.heappush(heap, (n, w))
                    elif (n, w) > heap[0]:
                        heapq.heapreplace(heap, (n, w))
        self.paracel_read_special_handle(self.handle_file, self.filter_function, handler)
        self.result = [(w, n) for n, w in sorted(heap, reverse=True)]

    def solve(self):
        lines = self.paracel_load(self.input)
        self.paracel_sync()
        self.learning(lines)
        self.paracel_sync()

    def print(self):
        if self.get_worker_id() == 0:
            for w, n in self.result:
                print(f"{w} : {n}")
