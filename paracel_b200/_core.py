"""Loader of the compiled host runtime ``_pcl_core`` (built in-tree by
``paracel_b200._build``; built on first use when it is missing)."""
from __future__ import annotations

import importlib.util
import sys

from . import _build

_mod = None


def core():
    global _mod
    if _mod is not None:
        return _mod
    path = _build.core_path()
    if not path.exists():
        _build.build_core()
    spec = importlib.util.spec_from_file_location("_pcl_core", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_pcl_core"] = mod
    _mod = mod
    return mod
