"""Ball tree for maximum-inner-product search (reference: tool/balltree/balltree.hpp and its
Cython wrapper balltree.pyx: ``PyQuery``, ``PyBalltree``, ``balltree_search``,
``linear_search`` and their ``_with_dp`` forms).  The tree itself is native
(``csrc/core/balltree.hpp``); ``search_batch_gpu`` answers many queries at once on the GPU by
brute force over the tcgen05 GEMM, which is the faster path for large batches."""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

import numpy as np

from .._core import core


class PyQuery:
    def __init__(self, item: Sequence[float], k: int = 1, black_list: Iterable[int] = (),
                 white_list: Iterable[int] = ()):
        self.item = [float(x) for x in item]
        self.k = int(k) if k else 1
        self.black = set(int(x) for x in black_list)
        self.white = set(int(x) for x in white_list)

    def get_k(self) -> int:
        return self.k

    def get_item(self) -> List[float]:
        return self.item

    def get_blacklist(self):
        return self.black

    def get_whitelist(self):
        return self.white


class PyBalltree:
    def __init__(self, items, limit: int = 20):
        self.items = np.ascontiguousarray(items, dtype=np.float64)
        self._t = core().BallTree(self.items, limit)

    def build(self):
        self._t.build()

    def pickle(self, fn: str):
        self._t.pickle(fn)

    def build_from_file(self, fn: str):
        self._t.unpickle(fn)

    @property
    def node_count(self) -> int:
        return self._t.node_count

    @property
    def last_visited(self) -> int:
        return self._t.last_visited


def balltree_search_with_dp(q: PyQuery, tree: PyBalltree) -> List[Tuple[int, float]]:
    return tree._t.search(q.item, q.k, q.black, q.white)


def balltree_search(q: PyQuery, tree: PyBalltree) -> List[int]:
    return [i for i, _ in balltree_search_with_dp(q, tree)]


def linear_search_with_dp(q: PyQuery, buf) -> List[Tuple[int, float]]:
    t = buf if isinstance(buf, PyBalltree) else PyBalltree(buf)
    return t._t.brute_force(q.item, q.k, q.black, q.white)


def linear_search(q: PyQuery, buf) -> List[int]:
    return [i for i, _ in linear_search_with_dp(q, buf)]


def search_batch_gpu(queries, items, k: int):
    """Top-k inner products for a batch of queries on the GPU: (indices, scores)."""
    import torch
    from ..ops.gemm import gemm_nt
    Q = torch.as_tensor(np.asarray(queries), dtype=torch.float32, device="cuda")
    X = torch.as_tensor(np.asarray(items), dtype=torch.float32, device="cuda")
    S = gemm_nt(Q, X, precise=True)
    sc, idx = torch.topk(S, k, dim=1)
    return idx.cpu().numpy(), sc.cpu().numpy()
