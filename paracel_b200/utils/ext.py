"""String and file helpers (reference: include/utils/ext_utility.hpp:38-221)."""
from __future__ import annotations

import glob as _glob
import os
import re
import time
from typing import Dict, Iterable, List, Sequence, Union


def str_split(s: str, seps: str) -> List[str]:
    """Split on a character or on any character of ``seps``; empty fields are dropped."""
    if len(seps) == 1:
        return [x for x in s.split(seps) if x]
    out, cur = [], []
    sset = set(seps)
    for ch in s:
        if ch in sset:
            if cur:
                out.append("".join(cur))
                cur = []
        else:
            cur.append(ch)
    if cur:
        out.append("".join(cur))
    return out


def str_split_by_word(s: str, seps: str) -> List[str]:
    """Split on a regular expression (a whole word such as ``_PARACEL_``); a trailing
    empty field is dropped."""
    out = re.split(seps, s)
    if out and out[-1] == "":
        out.pop()
    return out


def str_join(lst: Sequence[str], sep: str) -> str:
    return sep.join(lst)


def startswith(s: str, key: str) -> bool:
    return s.startswith(key)


def endswith(s: str, key: str) -> bool:
    return s.endswith(key)


def isfile(f: str) -> bool:
    return os.path.isfile(f)


def isdir(d: str) -> bool:
    return os.path.isdir(d)


def paracel_glob(pattern: str) -> List[str]:
    return sorted(_glob.glob(os.path.expanduser(pattern)))


def expand_dir_rec(dname: str) -> List[str]:
    out: List[str] = []
    for name in paracel_glob(todir(dname) + "*"):
        if isfile(name):
            out.append(name)
        else:
            out.extend(expand_dir_rec(name))
    return out


def expand(fname: Union[str, Iterable[str]]) -> List[str]:
    """A file, a directory (recursive), a glob pattern, or a list of those."""
    if not isinstance(fname, str):
        out: List[str] = []
        for f in fname:
            out.extend(expand(f))
        return out
    if isfile(fname):
        return [fname]
    if isdir(fname):
        return expand_dir_rec(fname)
    return paracel_glob(fname)


def dot_product(a: Sequence[float], b: Sequence[float]) -> float:
    return float(sum(x * y for x, y in zip(a, b)))


def todir(f: str) -> str:
    return f if f.endswith("/") else f + "/"


def add_folder_suffix_with_date(folder: str) -> str:
    now = time.localtime()
    suffix = f"{now.tm_year}{now.tm_mon}{now.tm_mday}"
    base = folder[:-1] if folder.endswith("/") else folder
    return base + suffix + "/"


def file_replace(src: str, dst: str, rep: Dict[str, str]) -> None:
    """Copy ``src`` to ``dst`` replacing every key of ``rep``; lines starting with '#' are dropped."""
    with open(src) as fin, open(dst, "w") as fout:
        for line in fin:
            line = line.rstrip("\n")
            if line.startswith("#"):
                continue
            for k, v in rep.items():
                line = line.replace(k, v)
            fout.write(line + "\n")
