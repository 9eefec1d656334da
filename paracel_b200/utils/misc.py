"""General helpers (reference: include/utils.hpp:116-334)."""
from __future__ import annotations

import json
import os
import random as _random
from typing import Any, Callable, Dict, List, Sequence

from .ext import expand
from .types import SEPERATOR


def random_double() -> float:
    """Uniform in the open interval (0, 1)."""
    v = _random.random()
    while v == 0.0 or v == 1.0:
        v = _random.random()
    return v


def random_double_list(n: int, upper_bnd: float = 1.0) -> List[float]:
    return [upper_bnd * random_double() for _ in range(n)]


class json_parser:
    """JSON configuration reader with dotted keys (``a.b``).  ``check_parse`` also
    verifies that the value names an existing file, directory or non-empty glob
    (include/utils.hpp:133-183)."""

    def __init__(self, fn: str):
        with open(fn) as f:
            self.pt = json.load(f)

    def _get(self, key: str):
        cur = self.pt
        for part in key.split("."):
            cur = cur[part]
        return cur

    def parse(self, key: str, typ: Callable = None):
        v = self._get(key)
        if typ is bool and isinstance(v, str):
            return v.lower() in ("1", "true", "yes")
        return typ(v) if typ is not None else v

    def check_parse(self, key: str, typ: Callable = None):
        v = self.parse(key, typ)
        if not expand(v):
            raise FileNotFoundError(f"config key {key}: {v} does not exist")
        return v

    def parse_v(self, key: str, typ: Callable = None) -> list:
        v = self._get(key)
        return [typ(x) if typ is not None else x for x in v]

    def check_parse_v(self, key: str, typ: Callable = None) -> list:
        v = self.parse_v(key, typ)
        for x in v:
            if not expand(x):
                raise FileNotFoundError(f"config key {key}: {x} does not exist")
        return v

    def get(self, key: str, default=None):
        try:
            return self._get(key)
        except (KeyError, TypeError):
            return default


def get_hostnames_dict(names: str) -> List[Dict[str, str]]:
    """``host:p0,p1,..`` entries joined by ``_PARACEL_`` -> list of {host, ports}."""
    out = []
    for item in names.split(SEPERATOR):
        if not item:
            continue
        host, ports = item.split(":", 1)
        out.append({"host": host, "ports": ports})
    return out


def cvt_id(x):
    """id <-> string conversion (include/utils.hpp:323-329)."""
    return str(x) if isinstance(x, int) else int(x)


def tail(filename: str, k: int, func: Callable[[str], Any] = lambda s: s) -> list:
    """Last ``k`` lines of a file mapped through ``func`` (ring buffer, include/utils.hpp:300-321)."""
    buf: List[Any] = []
    with open(filename) as f:
        for line in f:
            buf.append(func(line.rstrip("\n")))
            if len(buf) > k:
                buf.pop(0)
    return buf


def traverse_matrix(m, func: Callable[[int, int, float], None]) -> None:
    """Visit the stored entries of a scipy sparse matrix (or all entries of a dense one)."""
    try:
        import scipy.sparse as sp
        if sp.issparse(m):
            coo = m.tocoo()
            for i, j, v in zip(coo.row, coo.col, coo.data):
                func(int(i), int(j), float(v))
            return
    except ImportError:  # pragma: no cover
        pass
    for i in range(m.shape[0]):
        for j in range(m.shape[1]):
            func(i, j, float(m[i, j]))


def traverse_vector(v: Sequence[float], func: Callable[[int, float], None]) -> None:
    for i, x in enumerate(v):
        func(i, float(x))


def error_abort(msg: str) -> None:
    """Unlike the reference macro of the same name (which only prints) this raises."""
    raise RuntimeError(msg)
