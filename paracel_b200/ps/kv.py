"""Python face of the native KV table (reference: include/kv.hpp:29-173)."""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Tuple

from .._core import core
from ..utils.packer import pack, unpack


class kvs:
    def __init__(self):
        self._s = core().KVStore()

    def contains(self, k: str) -> bool:
        return self._s.contains(k)

    def set(self, k: str, v: Any) -> None:
        self._s.set(k, pack(v))

    def set_multi(self, d: Dict[str, Any]) -> None:
        self._s.set_multi({k: pack(v) for k, v in d.items()})

    def get(self, k: str, default: Any = None) -> Any:
        b = self._s.get(k)
        return default if b is None else unpack(b)

    def get_multi(self, keys: Iterable[str]) -> List[Any]:
        """Strict form: raises IndexError/KeyError when a key is missing."""
        return [unpack(b) for b in self._s.get_multi(list(keys))]

    def get_multi_dict(self, keys: Iterable[str]) -> Dict[str, Any]:
        return {k: unpack(b) for k, b in self._s.get_multi_existing(list(keys)).items()}

    def incr(self, k: str, delta: Any) -> bool:
        return self._s.incr(k, pack(delta))

    def gets(self, k: str) -> Optional[Tuple[Any, int]]:
        r = self._s.gets(k)
        if r is None:
            return None
        return unpack(r[0]), r[1]

    def cas(self, k: str, v: Any, uniq: int) -> bool:
        return self._s.cas(k, pack(v), uniq)

    def delete(self, k: str) -> bool:
        return self._s.delete(k)

    def clean(self) -> None:
        self._s.clean()

    def getall(self) -> Dict[str, Any]:
        return {k: unpack(b) for k, b in self._s.getall().items()}

    def __len__(self) -> int:
        return len(self._s)
