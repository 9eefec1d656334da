"""Key directory and store of the parameters that live in GPU memory.

The reference addresses every parameter by a string key and finds its server
with a consistent-hash ring (include/ps.hpp:434, include/ring.hpp:85-92).  The
device backend keeps the same keys visible -- ``"theta"``, ``"W_123"``,
``"usr_bias_7"``, ``"55_pr"``, a bare word id -- but maps a key to
``(table, row)`` by its pattern, and a row to its owner by arithmetic:

    exact key              -> DenseTable   (range-sharded fp32 vector)
    exact key              -> MatrixTable  (row-sharded matrix read through the fused gather+GEMM)
    prefix + id + suffix   -> RowTable     (fixed-width fp32 / int32 rows) or ScalarTable

``id`` is either the row number itself or, when the table was registered with
``names`` (the sorted original ids of the input file), the position of the id
in that array, so dumps and string keys carry the ids of the input.

The hot paths never format a string: a :class:`KeyBatch` stands for the keys
``prefix + str(id) + suffix`` of a whole id tensor and is accepted wherever the
``paralg`` API takes a list of keys.  Keys that match no registered pattern
belong to the host parameter server (any msgpack value), exactly as before.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import _lib
from .device_handlers import key_filter, resolve_device_handler
from .tables import DenseTable, RowTable, ScalarTable


class TableEntry:
    """One registered table: its key pattern, the table object and the optional id names."""

    def __init__(self, kind: str, table, prefix: str = "", suffix: str = "", key: str = "",
                 names=None, handler: str = "add"):
        self.kind, self.table = kind, table          # kind: rows | scalars | dense | matrix
        self.prefix, self.suffix, self.key = prefix, suffix, key
        self.handler = handler
        self.names = None if names is None else np.asarray(names)
        self._names_dev: Optional[torch.Tensor] = None

    @property
    def pattern(self) -> str:
        return self.key if self.kind in ("dense", "matrix") else f"{self.prefix}<id>{self.suffix}"

    # ---- string keys <-> rows (slow path: single keys, dumps, filters)
    def row_of(self, key: str) -> Optional[int]:
        """Row of a string key, or None if the key does not belong to this table."""
        if self.kind in ("dense", "matrix"):
            return 0 if key == self.key else None
        if not (key.startswith(self.prefix) and key.endswith(self.suffix)):
            return None
        body = key[len(self.prefix): len(key) - len(self.suffix) if self.suffix else None]
        if not body or not (body.isdigit() or (body[0] == "-" and body[1:].isdigit())):
            return None
        ident = int(body)
        if self.names is None:
            return ident if 0 <= ident < self.table.rows else None
        pos = int(np.searchsorted(self.names, ident))
        if pos >= self.names.size or int(self.names[pos]) != ident:
            return None
        return pos

    def key_of(self, row: int) -> str:
        if self.kind in ("dense", "matrix"):
            return self.key
        ident = row if self.names is None else int(self.names[row])
        return f"{self.prefix}{ident}{self.suffix}"

    def rows_of_ids(self, ids: torch.Tensor) -> torch.Tensor:
        """Rows of a tensor of original ids (identity without ``names``)."""
        if self.names is None:
            return ids
        if self._names_dev is None:
            self._names_dev = torch.as_tensor(self.names.astype(np.int64), device=self.table.device)
        return torch.searchsorted(self._names_dev, ids.to(self.table.device, torch.int64))


class KeyBatch:
    """The keys ``prefix + str(id) + suffix`` for every element of ``rows`` (int64 device tensor
    of table rows), as one object: the bulk argument of ``paracel_read_multi`` /
    ``paracel_write_multi`` / ``paracel_bupdate_multi`` on a device table."""

    __slots__ = ("entry", "rows")

    def __init__(self, entry: TableEntry, rows: torch.Tensor):
        self.entry = entry
        self.rows = _lib.check_cuda(rows, torch.int64, "rows")

    def __len__(self) -> int:
        return int(self.rows.numel())

    def keys(self) -> List[str]:
        """The key strings (host loop; for dumps and debugging, not for the training loop)."""
        return [self.entry.key_of(r) for r in self.rows.cpu().tolist()]


class MatrixTable:
    """Row-sharded fp32 matrix whose ``read`` is fused with the GEMM that consumes it
    (``paracel_b200.ops.gemm.DenseReadGemm``): the key's value is only ever seen as the
    product ``A @ value.T`` or the row-wise arg-min of it."""

    def __init__(self, rows: int, cols: int, group=None, device=None, kernel=None):
        from ..ops.gemm import DenseReadGemm
        self.g = DenseReadGemm(rows, cols, group, device, kernel=kernel)
        self.rows, self.cols = rows, cols
        self.device = self.g.device
        self.shard = self.g.shard

    def local_rows(self) -> Tuple[int, int]:
        return self.g.local_rows()

    def check(self):
        self.g.check()

    def free(self):
        self.shard = None
        self.g.free()


class DeviceStore:
    """All device tables of one ``paralg`` object plus the directory that finds them by key."""

    def __init__(self, group=None, device=None):
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        self.entries: List[TableEntry] = []
        self._exact: Dict[str, TableEntry] = {}

    # ------------------------------------------------------------ registration
    def _check_new(self, prefix: str, suffix: str, key: str):
        probe = key if key else f"{prefix}0{suffix}"
        if self.resolve(probe) is not None:
            raise ValueError(f"a device table already serves keys like {probe!r}")

    def add_rows(self, rows: int, width: int, prefix: str = "", suffix: str = "",
                 dtype=torch.float32, names=None, handler: str = "add") -> TableEntry:
        self._check_new(prefix, suffix, "")
        t = RowTable(rows, width, dtype, self.group, self.device)
        e = TableEntry("rows", t, prefix, suffix, names=names, handler=handler)
        self.entries.append(e)
        return e

    def add_scalars(self, rows: int, prefix: str = "", suffix: str = "", names=None,
                    handler: str = "add") -> TableEntry:
        self._check_new(prefix, suffix, "")
        t = ScalarTable(rows, self.group, self.device)
        e = TableEntry("scalars", t, prefix, suffix, names=names, handler=handler)
        self.entries.append(e)
        return e

    def add_dense(self, key: str, length: int, handler: str = "add", lr: float = 1.0,
                  lam: float = 0.0, timeout_s: float = 5.0) -> TableEntry:
        self._check_new("", "", key)
        resolve_device_handler(handler)
        t = DenseTable(length, self.group, self.device, handler=handler, lr=lr, lam=lam,
                       timeout_s=timeout_s)
        e = TableEntry("dense", t, key=key, handler=handler)
        self.entries.append(e)
        self._exact[key] = e
        return e

    def add_matrix(self, key: str, rows: int, cols: int, kernel=None) -> TableEntry:
        self._check_new("", "", key)
        e = TableEntry("matrix", MatrixTable(rows, cols, self.group, self.device, kernel), key=key)
        self.entries.append(e)
        self._exact[key] = e
        return e

    def drop(self, entry: TableEntry) -> None:
        """Unregister and free a table (collective)."""
        self.entries.remove(entry)
        self._exact.pop(entry.key, None)
        entry.table.free()

    # ---------------------------------------------------------------- look-up
    def resolve(self, key: str) -> Optional[Tuple[TableEntry, int]]:
        e = self._exact.get(key)
        if e is not None:
            return e, 0
        for e in self.entries:
            if e.kind in ("rows", "scalars"):
                r = e.row_of(key)
                if r is not None:
                    return e, r
        return None

    def batch(self, entry: TableEntry, ids, original_ids: bool = False) -> KeyBatch:
        """Key batch of ``entry`` for a tensor (or sequence) of rows; ``original_ids`` says that
        ``ids`` are ids of the input file to be translated through the table's ``names``."""
        t = torch.as_tensor(ids, dtype=torch.int64, device=self.device).contiguous()
        if original_ids:
            t = entry.rows_of_ids(t).contiguous()
        return KeyBatch(entry, t)

    def group_keys(self, keys: Sequence[str]):
        """Split string keys into per-table batches: ``([(entry, positions, KeyBatch)], host
        positions)``; positions index ``keys``."""
        per: Dict[int, Tuple[TableEntry, List[int], List[int]]] = {}
        host: List[int] = []
        for pos, k in enumerate(keys):
            hit = self.resolve(k)
            if hit is None:
                host.append(pos)
                continue
            e, r = hit
            slot = per.setdefault(id(e), (e, [], []))
            slot[1].append(pos)
            slot[2].append(r)
        out = [(e, pos, self.batch(e, rows)) for e, pos, rows in per.values()]
        return out, host

    # ------------------------------------------------------------------ reads
    def pull(self, kb: KeyBatch, out: Optional[torch.Tensor] = None,
             snapshot: Optional[torch.Tensor] = None, clock=None, target: int = 0) -> torch.Tensor:
        """Rows of a key batch into ``out`` (n x width, or n for scalars); the SSP wait for
        ``min clock >= target`` rides in the same kernel when ``clock`` is given."""
        e, t = kb.entry, kb.entry.table
        n = len(kb)
        if e.kind == "scalars":
            if out is None:
                out = torch.empty(n, device=self.device)
            if clock is not None and target > 0:
                clock.wait()
            t.pull(kb.rows, out, snapshot)
            return out
        if out is None:
            out = torch.empty(n, t.width, dtype=t.dtype, device=self.device)
        if clock is not None and target > 0 and t.dtype == torch.float32:
            t.pull(kb.rows, out, snapshot, clock.clocks, target, clock.timeout_ns, clock.status)
        else:
            if clock is not None and target > 0:
                clock.wait()
            t.pull(kb.rows, out, snapshot)
        return out

    def read_key(self, entry: TableEntry, row: int):
        """Value of one key: the whole vector of a dense key, one row (tensor) or one scalar."""
        if entry.kind == "dense":
            return entry.table.read()
        if entry.kind == "matrix":
            raise TypeError(f"{entry.key!r} is a matrix table: read it with paracel_read_matmul")
        kb = self.batch(entry, [row])
        out = self.pull(kb)
        return out[0].item() if entry.kind == "scalars" else out[0]

    # ----------------------------------------------------------------- writes
    def push(self, kb: KeyBatch, values: torch.Tensor, handler: Optional[str] = None,
             old: Optional[torch.Tensor] = None, wgt: Optional[torch.Tensor] = None,
             refresh_old: bool = True, start: int = 0, status=None) -> None:
        """``paracel_bupdate_multi`` of a key batch: reduce ``wgt * (values - old)`` (or
        ``values`` without a snapshot) into the owners' rows with the named handler."""
        e = kb.entry
        h = resolve_device_handler(handler or e.handler)
        if h.kind not in ("add", "scaled_add", "max", "assign"):
            raise ValueError(f"handler kind {h.kind!r} cannot run on a row table")
        kw = {}
        if e.kind == "rows":
            kw = {"scale": 1.0 if h.scale is None else h.scale, "start": start}
        e.table.push(kb.rows, values, old, wgt, handler=h.kind, refresh_old=refresh_old,
                     status=status, **kw)

    def write_key(self, entry: TableEntry, row: int, value) -> None:
        if entry.kind == "dense":
            v = torch.as_tensor(value, dtype=torch.float32, device=self.device).contiguous()
            entry.table.write(v)
            return
        if entry.kind == "matrix":
            raise TypeError(f"{entry.key!r} is a matrix table: owners write their shard")
        kb = self.batch(entry, [row])
        t = entry.table
        v = torch.as_tensor(value, dtype=t.dtype, device=self.device).reshape(1, -1).contiguous()
        if v.shape[1] != t.width:
            full = torch.zeros(1, t.width, dtype=t.dtype, device=self.device)
            full[:, : v.shape[1]] = v
            v = full
        self.push(kb, v.view(-1) if entry.kind == "scalars" else v, "assign")

    # ------------------------------------------------------------- whole tables
    def matching(self, file_name: str, func_name: str) -> List[TableEntry]:
        """Row / scalar / dense tables whose keys pass the filter.  The filter is evaluated on
        one key of each table: the filters are predicates on the key pattern (prefix, suffix),
        not on single ids."""
        f = key_filter(file_name, func_name)
        out = []
        for e in self.entries:
            if e.kind == "matrix":
                continue
            if e.kind == "dense":
                if f(e.key):
                    out.append(e)
            elif e.table.rows > 0 and f(e.key_of(0)):
                out.append(e)
        return out

    def dump_entry(self, entry: TableEntry, width: Optional[int] = None) -> Dict[str, Any]:
        """Every key of a table with its value, gathered from all owners over NVLink (key ->
        float for scalars, list for rows, list for a dense vector)."""
        if entry.kind == "dense":
            return {entry.key: entry.table.read().cpu().tolist()}
        t = entry.table
        rows = torch.arange(t.rows, dtype=torch.int64, device=self.device)
        vals = self.pull(KeyBatch(entry, rows))
        torch.cuda.synchronize(self.device)
        if entry.kind == "scalars":
            return dict(zip((entry.key_of(r) for r in range(t.rows)), vals.cpu().tolist()))
        v = vals[:, :width] if width else vals
        return dict(zip((entry.key_of(r) for r in range(t.rows)), v.cpu().tolist()))

    def check(self) -> None:
        for e in self.entries:
            e.table.check()

    def free(self) -> None:
        for e in self.entries:
            e.table.free()
        self.entries = []
        self._exact = {}
