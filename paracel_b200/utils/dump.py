"""Writers for the reference's key/value text dump layout.

Number formatting follows the two conventions the reference mixes
(include/ps.hpp:983-1228, 1308-1336): ``cvt(double)`` is ``std::to_string``
(fixed, six decimals) and a plain ``ostream << double`` is six significant
digits (``%g``).  Keys are written in sorted order (the reference iterates an
``unordered_map``, whose order is unspecified).  Empty containers write
nothing instead of underflowing ``size() - 1`` as the reference does.
"""
from __future__ import annotations

import io
import os
from typing import Dict, Sequence, Union

Sink = Union[str, io.TextIOBase]


def to_string(v) -> str:
    """``std::to_string`` for doubles and integers."""
    if isinstance(v, float):
        return "%.6f" % v
    if isinstance(v, bool):
        return "1" if v else "0"
    if isinstance(v, int):
        return str(v)
    if hasattr(v, "item"):
        return to_string(v.item())
    return str(v)


def ostream_double(v: float) -> str:
    """Default ``std::ostream << double`` (precision 6, %g-like)."""
    s = "%g" % float(v)
    return s


def cvt(v) -> str:
    """The overload set of ``paralg::cvt`` (ps.hpp:1308-1336)."""
    if isinstance(v, str):
        return v
    if isinstance(v, tuple) and len(v) == 3:
        return f"{to_string(v[0])},{to_string(v[1])},{to_string(float(v[2]))}"
    if isinstance(v, tuple) and len(v) == 2:
        a, b = v
        if isinstance(a, (list, tuple)):
            return ",".join(to_string(float(x)) for x in a) + ":" + to_string(float(b))
        return f"{to_string(a)}:{to_string(float(b))}"
    if isinstance(v, int):
        return str(v)
    return to_string(float(v))


def _open(sink: Sink, append: bool):
    if isinstance(sink, str):
        d = os.path.dirname(sink)
        if d:
            os.makedirs(d, exist_ok=True)
        return open(sink, "a" if append else "w"), True
    return sink, False


def _sorted_items(d: Dict):
    try:
        return sorted(d.items(), key=lambda kv: kv[0])
    except TypeError:
        return sorted(d.items(), key=lambda kv: str(kv[0]))


def dump_vector(data: Sequence, sink: Sink, sep: str = ",", append: bool = False):
    f, close = _open(sink, append)
    if len(data) > 0:
        f.write(sep.join(cvt(x) for x in data) + "\n")
    if close:
        f.close()


def dump_dict_scalar(data: Dict, sink: Sink, append: bool = False):
    """``key\\tvalue`` with ints verbatim and doubles as ostream doubles."""
    f, close = _open(sink, append)
    for k, v in _sorted_items(data):
        if isinstance(v, float):
            f.write(f"{k}\t{ostream_double(v)}\n")
        else:
            f.write(f"{k}\t{v}\n")
    if close:
        f.close()


def dump_dict_vector(data: Dict, sink: Sink, append: bool = False):
    """``key\\tcvt(p0)|cvt(p1)|...`` (ps.hpp:1081-1116)."""
    f, close = _open(sink, append)
    for k, lst in _sorted_items(data):
        if len(lst) == 0:
            continue
        f.write(f"{k}\t" + "|".join(cvt(x) for x in lst) + "\n")
    if close:
        f.close()


def dump_dict_pairs(data: Dict, sink: Sink, append: bool = False):
    """``key\\tk0:v0|k1:v1`` with values through std::to_string (ps.hpp:1118-1194)."""
    f, close = _open(sink, append)
    for k, lst in _sorted_items(data):
        if len(lst) == 0:
            continue
        f.write(f"{k}\t" + "|".join(f"{a}:{to_string(float(b))}" for a, b in lst) + "\n")
    if close:
        f.close()


def dump_prob_mtx(data: Dict, sink: Sink, append: bool = False):
    """Like :func:`dump_dict_pairs` but the last value is an ostream double and a key
    with an empty list still writes ``key\\t`` (ps.hpp:1196-1228)."""
    f, close = _open(sink, append)
    for k, lst in _sorted_items(data):
        f.write(f"{k}\t")
        if len(lst) == 0:
            continue
        head = [f"{a}:{to_string(float(b))}" for a, b in lst[:-1]]
        a, b = lst[-1]
        head.append(f"{a}:{ostream_double(b)}")
        f.write("|".join(head) + "\n")
    if close:
        f.close()


def read_dict_vector(path: str, sep: str = "|") -> Dict[str, list]:
    out = {}
    with open(path) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            k, v = line.split("\t", 1)
            out[k] = [float(x) for x in v.split(sep) if x != ""]
    return out


def read_dict_scalar(path: str) -> Dict[str, float]:
    out = {}
    with open(path) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            k, v = line.split("\t", 1)
            out[k] = float(v)
    return out


def files_merge(pattern: str, out_path: str):
    """Concatenate the per-rank files matching ``pattern`` (ps.hpp:948-972)."""
    import glob
    names = sorted(n for n in glob.glob(pattern) if not n.endswith("merge"))
    with open(out_path, "w") as out:
        for n in names:
            with open(n) as f:
                out.write(f.read())
