"""Serialisation of parameter values (reference: include/packer.hpp:39-75).

Values travel and are stored as msgpack byte strings.  ``pack``/``unpack`` are
the plain forms; ``pack_prefixed``/``unpack_prefixed`` add the leading native
``size_t`` length the reference writes in front of a body when it packs into a
``std::string`` (used by the ``pkl_dat`` files).  Numpy arrays and torch tensors
are packed as (nested) lists, tuples as lists, sets as lists.
"""
from __future__ import annotations

import struct
from typing import Any

import msgpack
import numpy as np


def _default(o):
    if isinstance(o, np.ndarray):
        return o.tolist()
    if isinstance(o, (np.integer,)):
        return int(o)
    if isinstance(o, (np.floating,)):
        return float(o)
    if isinstance(o, (set, frozenset)):
        return sorted(o)
    if hasattr(o, "detach") and hasattr(o, "cpu"):
        return o.detach().cpu().tolist()
    if hasattr(o, "to_packable"):
        return o.to_packable()
    raise TypeError(f"cannot pack {type(o)}")


def pack(v: Any) -> bytes:
    return msgpack.packb(v, default=_default, use_bin_type=True)


def unpack(b: bytes) -> Any:
    return msgpack.unpackb(b, raw=False, strict_map_key=False)


def pack_prefixed(v: Any) -> bytes:
    body = pack(v)
    return struct.pack("<Q", len(body)) + body


def unpack_prefixed(b: bytes) -> Any:
    (n,) = struct.unpack("<Q", b[:8])
    return unpack(b[8:8 + n])


class packer:
    """Object form kept for API familiarity: ``packer(v).pack()`` / ``packer().unpack(b)``."""

    def __init__(self, val: Any = None):
        self.val = val

    def pack(self) -> bytes:
        return pack(self.val)

    def unpack(self, b: bytes) -> Any:
        return unpack(b)


def pkl_dat_sequential(data: Any, path: str) -> None:
    """Write ``data`` as one length-prefixed msgpack blob (include/utils.hpp:336-365).
    2-D numpy arrays are stored column-major as a flat list; scipy sparse matrices as a
    list of ((i, j), v)."""
    try:
        import scipy.sparse as sp
    except Exception:  # pragma: no cover
        sp = None
    if sp is not None and sp.issparse(data):
        coo = data.tocoo()
        data = [[[int(i), int(j)], float(v)] for i, j, v in zip(coo.row, coo.col, coo.data)]
    elif isinstance(data, np.ndarray) and data.ndim == 2:
        data = data.flatten(order="F").tolist()
    with open(path, "wb") as f:
        f.write(pack_prefixed(data))


def unpkl_dat_sequential(path: str, cols: int = 0, sparse: bool = False):
    with open(path, "rb") as f:
        v = unpack_prefixed(f.read())
    if sparse:
        import scipy.sparse as sp
        if not v:
            return sp.csr_matrix((0, 0))
        rows = [p[0][0] for p in v]
        colsv = [p[0][1] for p in v]
        vals = [p[1] for p in v]
        return sp.csr_matrix((vals, (rows, colsv)))
    if cols:
        a = np.asarray(v, dtype=np.float64)
        return a.reshape((cols, -1)).T.copy() if a.size else a.reshape(0, cols)
    return v
