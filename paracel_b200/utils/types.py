"""Constants and small container types (reference: include/paracel_types.hpp:43-61
constants, 256-304 ``bag_type``)."""
from __future__ import annotations

from typing import Callable, Generic, Iterable, Iterator, List, TypeVar

BLK_SZ = 32            # byte blocks per worker for the map-style load patterns
THREADS_NUM = 5        # op classes of a client connection set
SEPERATOR = "_PARACEL_"          # separator of server endpoint lists (spelling as in the reference)
SEPERATOR_INNER = "_ps_"
DEFAULT_PORT = 11777
SENTINEL = 2147483648  # "no out-link" marker in PageRank inputs (pr.hpp:28)

T = TypeVar("T")


class bag_type(Generic[T]):
    """A growable bag of items with ``put``, ``get`` (copy), ``traverse`` and iteration."""

    def __init__(self, items: Iterable[T] = ()):
        self.c: List[T] = list(items)

    def put(self, item: T) -> None:
        self.c.append(item)

    def get(self) -> "bag_type[T]":
        return bag_type(self.c)

    def is_empty(self) -> bool:
        return not self.c

    def size(self) -> int:
        return len(self.c)

    def __len__(self) -> int:
        return len(self.c)

    def traverse(self, func: Callable[[T], None]) -> None:
        for x in self.c:
            func(x)

    def __iter__(self) -> Iterator[T]:
        return iter(self.c)

    def assign(self, other: "bag_type[T]") -> "bag_type[T]":
        """Copy-assignment that returns ``self`` (the reference's operator= forgets to)."""
        self.c = list(other.c)
        return self


# (row id, column id, weight) as produced by the loader; the "compact" form has dense int ids
triple_type = tuple
compact_triple_type = tuple
threads_num = THREADS_NUM


def is_comm_builtin(v) -> bool:
    """Scalars that travel as one fixed-size element (paracel_types.hpp:63-118)."""
    return isinstance(v, (bool, int, float))


def is_comm_container(v) -> bool:
    """Flat containers of builtin scalars (or a string) that travel as size + payload."""
    if isinstance(v, (str, bytes)):
        return True
    try:
        import numpy as np
        if isinstance(v, np.ndarray):
            return v.ndim == 1
    except ImportError:  # pragma: no cover
        pass
    return isinstance(v, (list, tuple)) and all(is_comm_builtin(x) for x in v)


def is_matrix(v) -> bool:
    """Dense 2-D arrays and scipy sparse matrices."""
    try:
        import numpy as np
        if isinstance(v, np.ndarray):
            return v.ndim == 2
        import scipy.sparse as sp
        return bool(sp.issparse(v))
    except ImportError:  # pragma: no cover
        return False


def is_atomic(v) -> bool:
    return isinstance(v, (bool, int, float, str))


def is_seqic(v) -> bool:
    return isinstance(v, (list, tuple)) and all(isinstance(x, (int, float)) for x in v)
