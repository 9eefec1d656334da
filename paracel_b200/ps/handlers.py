"""Update handlers and filters of the host parameter server.

The reference registers handlers as ``extern "C"`` objects made by
``update_proxy`` / ``filter_with_key_proxy`` and loads them with ``dlopen``
from the path given in ``update_file`` (include/proxy.hpp:32-73,
include/server.hpp:177-191).  Here a handler is named by ``(file, func)`` too:

* ``func`` is the name of a built-in kind implemented natively (``add``,
  ``max``, ``concat``, ... and every handler name the reference ships, e.g.
  ``lr_theta_update``, ``mf_fac_updater``, ``max_updater``);
* or ``file`` is a ``.py`` file (or importable module name) that defines a
  function ``func(old, delta) -> new`` on unpacked values -- the server
  imports it once and caches it;
* or ``file`` is a ``.so`` exporting ``func`` with the C ABI documented in
  ``csrc/core/ps_server.hpp``;
* filters are ``prefix:<p>``, ``suffix:<s>``, ``contains:<c>``, a filter name
  shipped with the reference, or a Python function ``func(key) -> bool``
  (``func(key, value)`` for the two-argument form).
"""
from __future__ import annotations

import importlib
import importlib.util
import inspect
import os
import sys
from typing import Any, Callable, Dict, Tuple

from ..utils.packer import pack, unpack

import threading

_PY_CACHE: Dict[Tuple[str, str], Callable] = {}
_LOCAL: Dict[str, Callable] = {}
_LOAD_LOCK = threading.Lock()


def register_handler(name: str, fn: Callable) -> None:
    """Make ``fn`` available under ``name`` to servers running in this process."""
    _LOCAL[name] = fn


def _load(file: str, func: str) -> Callable:
    key = (file, func)
    if key in _PY_CACHE:
        return _PY_CACHE[key]
    with _LOAD_LOCK:  # server threads may ask for the same file at the same time
        return _load_locked(file, func, key)


def _load_locked(file: str, func: str, key) -> Callable:
    if key in _PY_CACHE:
        return _PY_CACHE[key]
    if func in _LOCAL and not file:
        fn = _LOCAL[func]
    elif file.endswith(".py") and os.path.exists(file):
        modname = "_pcl_handlers_" + str(abs(hash(os.path.abspath(file))))
        if modname in sys.modules:
            mod = sys.modules[modname]
        else:
            spec = importlib.util.spec_from_file_location(modname, file)
            mod = importlib.util.module_from_spec(spec)
            sys.modules[modname] = mod
            spec.loader.exec_module(mod)
        fn = getattr(mod, func)
    elif file:
        mod = importlib.import_module(file)
        fn = getattr(mod, func)
    elif func in _LOCAL:
        fn = _LOCAL[func]
    else:
        raise KeyError(f"no handler named {func!r} (file {file!r})")
    _PY_CACHE[key] = fn
    return fn


def update_proxy(fn: Callable[[Any, Any], Any]) -> Callable[[bytes, bytes], bytes]:
    """Lift ``f(old, delta) -> new`` to packed values (include/proxy.hpp:56-73)."""
    def proxy(old: bytes, delta: bytes) -> bytes:
        return pack(fn(unpack(old), unpack(delta)))
    return proxy


def filter_proxy(fn: Callable[[str, Any], bool]) -> Callable[[str, bytes], bool]:
    def proxy(key: str, val: bytes) -> bool:
        return bool(fn(key, unpack(val)))
    return proxy


def filter_with_key_proxy(fn: Callable[[str], bool]) -> Callable[[str, bytes], bool]:
    def proxy(key: str, val: bytes) -> bool:
        return bool(fn(key))
    return proxy


def python_update_callback(file: str, func: str, old: bytes, delta: bytes) -> bytes:
    return pack(_load(file, func)(unpack(old), unpack(delta)))


def python_filter_callback(file: str, func: str, key: str, val: bytes) -> bool:
    fn = _load(file, func)
    try:
        nargs = len(inspect.signature(fn).parameters)
    except (TypeError, ValueError):
        nargs = 1
    if nargs >= 2:
        return bool(fn(key, unpack(val)))
    return bool(fn(key))
