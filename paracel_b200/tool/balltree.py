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


class DeviceBalltree:
    """A built ball tree copied to the GPU for batched search (csrc/cuda/balltree.cu)."""

    def __init__(self, tree: PyBalltree, device=None):
        import torch
        dev = torch.device(device if device is not None else "cuda")
        mu, rad, child, rng, order = tree._t.export_arrays()
        self.dim = tree.items.shape[1]
        self.n = tree.items.shape[0]
        self.child = torch.as_tensor(np.asarray(child, dtype=np.int32), device=dev)
        self.range = torch.as_tensor(np.asarray(rng, dtype=np.int64), device=dev)
        self.radius = torch.as_tensor(np.asarray(rad, dtype=np.float32), device=dev)
        self.mu = torch.as_tensor(np.asarray(mu, dtype=np.float32).reshape(-1, self.dim), device=dev)
        order = np.asarray(order, dtype=np.int64)
        self.ids = torch.as_tensor(order, device=dev)
        self.items = torch.as_tensor(tree.items[order].astype(np.float32), device=dev).contiguous()
        self.device = dev
        # the search kernel follows these indices without checking them again (an unpickled tree
        # could be damaged): child links are -1 or a node, item ranges lie inside the item array
        from ..ops import _lib
        _lib.validate_ids(self.child.view(-1), 0, self.radius.numel(), "ball tree (child links)", skip=-1)
        _lib.validate_ids(self.range.view(-1), 0, self.n + 1, "ball tree (item ranges)")

    def search(self, queries, k: int = 1):
        """(indices [nq, k], scores [nq, k], balls opened [nq]) for a batch of queries; queries
        whose traversal overflowed the device stack are answered by a dense product instead."""
        import torch
        from ..ops import _lib
        if not 1 <= k <= 32:
            raise ValueError("device search supports 1 <= k <= 32")
        if isinstance(queries, torch.Tensor):
            Q = queries.to(self.device, torch.float32).contiguous()
        else:
            Q = torch.as_tensor(np.asarray(queries, dtype=np.float32), device=self.device).contiguous()
        nq = Q.shape[0]
        idx = torch.empty(nq, k, dtype=torch.int64, device=self.device)
        sc = torch.empty(nq, k, dtype=torch.float32, device=self.device)
        vis = torch.empty(nq, dtype=torch.int32, device=self.device)
        _lib.call("pcl_balltree_search", self.child, self.range, self.radius, self.mu, self.items, self.ids,
                  Q, self.dim, nq, k, idx, sc, vis, _lib.stream_ptr())
        bad = torch.nonzero(vis < 0).flatten()
        if bad.numel():
            S = Q[bad] @ self.items.T
            s2, j2 = torch.topk(S, min(k, self.n), dim=1)
            idx[bad, : j2.shape[1]] = self.ids[j2]
            sc[bad, : j2.shape[1]] = s2
        return idx, sc, vis


def search_batch_gpu(queries, items, k: int):
    """Top-k inner products for a batch of queries on the GPU: (indices, scores)."""
    import torch
    from ..ops.gemm import gemm_nt
    Q = torch.as_tensor(np.asarray(queries), dtype=torch.float32, device="cuda")
    X = torch.as_tensor(np.asarray(items), dtype=torch.float32, device="cuda")
    S = gemm_nt(Q, X, precise=True)
    sc, idx = torch.topk(S, k, dim=1)
    return idx.cpu().numpy(), sc.cpu().numpy()
