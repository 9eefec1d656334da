"""Client side of the host parameter server: one ``kvclt`` per server
(reference: include/client.hpp:35-629).  Like the reference it keeps one
connection per operation class (read / push / update / bupdate / SSP ints), so a
non-blocking ``update`` never queues behind a blocking read.  A missing key is
reported as ``KeyError`` (the reference's "nokey" sentinel)."""
from __future__ import annotations

import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Dict, List, Optional, Sequence

import msgpack

from .._core import core
from ..utils.packer import pack, unpack

ST_OK, ST_NOKEY, ST_ERROR = 0, 1, 2


class PsError(RuntimeError):
    pass


class kvclt:
    _CLASSES = ("read", "push", "update", "bupdate", "ssp")

    def __init__(self, host: str, port: int, timeout_s: float = 0.0, inproc=None):
        self.host, self.port, self.timeout_s = host, int(port), timeout_s
        self._conns: Dict[str, Any] = {}
        self._lock = threading.Lock()
        self._inproc = inproc  # a PsServer object: call it without sockets
        self._pool: Optional[ThreadPoolExecutor] = None

    # ---------------------------------------------------------------- wire
    def _conn(self, cls: str):
        with self._lock:
            c = self._conns.get(cls)
            if c is None:
                c = core().PsConnection(self.host, self.port, self.timeout_s)
                self._conns[cls] = c
            return c

    def _call(self, cls: str, *fields) -> Any:
        req = msgpack.packb(list(fields), use_bin_type=True)
        if self._inproc is not None:
            rep = self._inproc.execute(req)
        else:
            rep = self._conn(cls).request(req)
        status, payload = msgpack.unpackb(rep, raw=False, strict_map_key=False)
        if status == ST_NOKEY:
            raise KeyError(fields[1] if len(fields) > 1 else "nokey")
        if status != ST_OK:
            raise PsError(str(payload))
        return payload

    def close(self):
        with self._lock:
            for c in self._conns.values():
                c.close()
            self._conns.clear()
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None

    # --------------------------------------------------------------- reads
    def contains(self, key: str) -> bool:
        return bool(self._call("read", "contains", key))

    def pull(self, key: str) -> Any:
        return unpack(self._call("read", "pull", key))

    def pull_multi(self, keys: Sequence[str]) -> List[Any]:
        return [unpack(b) for b in self._call("read", "pull_multi", list(keys))]

    def pull_multi_check(self, keys: Sequence[str]) -> Dict[str, Any]:
        return {k: unpack(v) for k, v in self._call("read", "pull_multi_check", list(keys)).items()}

    def pullall(self) -> Dict[str, Any]:
        return {k: unpack(v) for k, v in self._call("read", "pullall").items()}

    def pullall_raw(self) -> Dict[str, bytes]:
        return dict(self._call("read", "pullall"))

    def pullall_special(self, file: str = "", func: str = "") -> Dict[str, Any]:
        args = (file, func) if func else ()
        return {k: unpack(v) for k, v in self._call("read", "pullall_special", *args).items()}

    def register_pullall_special(self, file: str, func: str) -> bool:
        return bool(self._call("read", "register_pullall_special", file, func))

    def register_remove_special(self, file: str, func: str) -> bool:
        return bool(self._call("read", "register_remove_special", file, func))

    def register_update(self, file: str, func: str) -> bool:
        return bool(self._call("update", "register_update", file, func))

    def register_bupdate(self, file: str, func: str) -> bool:
        return bool(self._call("bupdate", "register_bupdate", file, func))

    # -------------------------------------------------------------- writes
    def push(self, key: str, val: Any) -> bool:
        return bool(self._call("push", "push", key, pack(val)))

    def push_multi(self, kvs: Dict[str, Any]) -> bool:
        keys = list(kvs.keys())
        return bool(self._call("push", "push_multi", keys, [pack(kvs[k]) for k in keys]))

    def bupdate(self, key: str, delta: Any, file: str = "", func: str = "") -> Any:
        args = (file, func) if func else ()
        return unpack(self._call("bupdate", "bupdate", key, pack(delta), *args))

    def bupdate_multi(self, keys: Sequence[str], deltas: Sequence[Any], file: str = "",
                      func: str = "") -> List[Any]:
        args = (file, func) if func else ()
        out = self._call("bupdate", "bupdate_multi", list(keys), [pack(d) for d in deltas], *args)
        return [unpack(b) for b in out]

    def update(self, key: str, delta: Any, file: str = "", func: str = "") -> Future:
        """Non-blocking update: returns a future of the success flag (client.hpp:257-291)."""
        if self._pool is None:
            self._pool = ThreadPoolExecutor(max_workers=1)
        args = (file, func) if func else ()
        packed = pack(delta)

        def run():
            self._call("update", "update", key, packed, *args)
            return True
        return self._pool.submit(run)

    def remove(self, key: str) -> bool:
        return bool(self._call("read", "remove", key))

    def remove_special(self, file: str = "", func: str = "") -> bool:
        args = (file, func) if func else ()
        return bool(self._call("read", "remove_special", *args))

    def clear(self) -> bool:
        return bool(self._call("read", "clear"))

    def size(self) -> int:
        return int(self._call("read", "size"))

    # ------------------------------------------------------------ SSP ints
    def push_int(self, key: str, val: int) -> bool:
        return bool(self._call("ssp", "push_int", key, int(val)))

    def incr_int(self, key: str, delta: int) -> bool:
        return bool(self._call("ssp", "incr_int", key, int(delta)))

    def pull_int(self, key: str) -> int:
        return int(self._call("ssp", "pull_int", key))

    def ssp_commit(self, clock: int) -> int:
        return int(self._call("ssp", "ssp_commit", int(clock)))

    def ssp_depart(self) -> int:
        return int(self._call("ssp", "ssp_depart"))

    def ssp_reset(self, worker_sz: int) -> bool:
        return bool(self._call("ssp", "ssp_reset", int(worker_sz)))

    def ping(self) -> str:
        return self._call("read", "ping")

    def shutdown(self) -> bool:
        return bool(self._call("read", "shutdown"))
