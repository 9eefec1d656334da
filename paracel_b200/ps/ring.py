"""Consistent-hash ring over server ids (reference: include/ring.hpp:35-98)."""
from __future__ import annotations

from typing import Any, Dict, Iterable

from .._core import core


class ring:
    def __init__(self, names: Iterable[Any], replicas: int = 32):
        self._r = core().Ring(replicas)
        self._names: Dict[str, Any] = {}
        for n in names:
            self.add_server(n)

    def add_server(self, name: Any) -> None:
        self._names[str(name)] = name
        self._r.add_server(str(name))

    def remove_server(self, name: Any) -> None:
        self._names.pop(str(name), None)
        self._r.remove_server(str(name))

    def get_server(self, key: Any) -> Any:
        """Server that owns ``key`` (strings hash as std::hash<std::string>, integers as
        themselves, like the C++ standard library does)."""
        c = core()
        if isinstance(key, str):
            h = c.hash_string(key)
        elif isinstance(key, int):
            h = c.hash_u64(key & 0xFFFFFFFFFFFFFFFF)
        elif isinstance(key, float):
            h = c.hash_double(key)
        else:
            h = c.hash_string(str(key))
        return self._names[self._r.get_server_by_hash(h)]
