"""``paracel::utils::hash<T>`` (include/utils/hash.hpp:37-92): ``std::hash`` for scalars and strings,
the "vechash" string hash for lists and a CityHash-style ``hash_combine`` for pairs.  The values are
those of libstdc++ on x86-64, so key placement (ring, loader grid) matches a reference build there."""
from __future__ import annotations

from typing import Any

from .._core import core


def hash_combine(x: int, y: int) -> int:
    """Mix of two 64-bit hash values (utils/hash.hpp:52-63)."""
    return core().hash_value_combine(x & 0xFFFFFFFFFFFFFFFF, y & 0xFFFFFFFFFFFFFFFF)


def hash_value(v: Any) -> int:
    c = core()
    if isinstance(v, bool):
        return int(v)
    if isinstance(v, int):
        return c.hash_u64(v & 0xFFFFFFFFFFFFFFFF)
    if isinstance(v, float):
        return c.hash_double(v)
    if isinstance(v, str):
        return c.hash_string(v)
    if isinstance(v, bytes):
        return c.hash_bytes(v)
    if isinstance(v, tuple) and len(v) == 2:
        return hash_combine(hash_value(v[0]), hash_value(v[1]))
    if isinstance(v, (list, tuple)):
        return c.hash_string_list([str(x) for x in v])
    raise TypeError(f"no hash for {type(v).__name__}")
