"""General helpers (reference: include/utils.hpp:116-334)."""
from __future__ import annotations

import json
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


ERROR_ABORT = error_abort


def error_print(msg: str) -> None:
    """ERROR_PRINT of the reference (include/utils.hpp:45-47): message to stderr, no exception."""
    import sys
    print(msg, file=sys.stderr)


def get_hostnames_string(srv_num: int, init_port: str = "") -> str:
    """Server side of the rendezvous (include/utils.hpp:58-77): listen on ``init_port`` for one
    ``host:p0,p1,..`` line from each of ``srv_num`` servers and return them joined by the
    endpoint separator.  The native implementation is the one the launcher uses."""
    from .._core import core
    from .types import DEFAULT_PORT
    port = int(init_port) if init_port else DEFAULT_PORT
    return SEPERATOR.join(core().collect_endpoints("0.0.0.0", port, srv_num, 600.0, None))


def is_idle_port(port: int) -> bool:
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        try:
            s.bind(("", port))
            return True
        except OSError:
            return False


def gen_port() -> int:
    """A port in [2014, 65535) that is free right now (the reference's probe always says yes,
    include/utils.hpp:94-105; this one really binds)."""
    import random
    for _ in range(1000):
        p = random.randrange(2014, 65535)
        if is_idle_port(p):
            return p
    raise RuntimeError("no idle port found")


def get_ports(n: int = None) -> List[int]:
    from .types import THREADS_NUM
    return [gen_port() for _ in range(THREADS_NUM if n is None else n)]


class heap_node:
    """(value, key) ordered by value: the element type of the top-k min-heaps (utils.hpp:270-276)."""
    __slots__ = ("val", "key")

    def __init__(self, key, val):
        self.key, self.val = key, val

    def __lt__(self, other):
        return self.val < other.val

    def __repr__(self):
        return f"heap_node({self.key!r}, {self.val!r})"


def cheat_to_os() -> None:
    """The reference touches a dummy std::thread so that libpthread is linked (utils.hpp:278-280);
    nothing to do here."""


def vec2evec(v: Sequence[float]):
    import numpy as np
    return np.asarray(v, dtype=np.float64)


def evec2vec(ev) -> List[float]:
    return [float(x) for x in ev]


def mat2vec(m) -> List[float]:
    """Column-major flattening, as Eigen stores a MatrixXd (utils.hpp:244-256)."""
    import numpy as np
    return np.asarray(m, dtype=np.float64).flatten(order="F").tolist()


def vec2mat(v: Sequence[float], rows: int):
    import numpy as np
    a = np.asarray(v, dtype=np.float64)
    return a.reshape((rows, a.size // rows), order="F")


def ring_bsearch(data: Sequence[int], key: int) -> int:
    """Index of the first ring point >= key, 0 when key is outside the ring (utils.hpp:282-298)."""
    import bisect
    if not data or key < data[0] or key > data[-1]:
        return 0
    return bisect.bisect_left(data, key)


def wait(future) -> bool:
    """Block on the future of a non-blocking update (utils.hpp:331-334)."""
    return future.result() if hasattr(future, "result") else bool(future)
