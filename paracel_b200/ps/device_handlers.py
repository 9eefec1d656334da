"""Update handlers and key filters of the tables that live in GPU memory.

The reference names a server-side handler by ``(update_file, func_name)`` and
loads it with ``dlopen`` (include/server.hpp:177-191, include/proxy.hpp:56-73).
On the device a handler is one of the reduction kinds that the push / bupdate
kernels implement at the owner of a row (``csrc/cuda/rows.cu``,
``csrc/cuda/dense.cu``), selected by the same ``func_name`` strings:

    add         new = old + delta                      (every *_incr_*, lr_theta_update, ...)
    scaled_add  new = old + scale * delta
    sgd         new = old - lr * delta
    prox_l1     w = old - lr * delta; new = sign(w) * max(|w| - |lr| * lam, 0)
    max         new = max(old, delta)                  (max_updater)
    assign      new = delta                            (paracel_write)

``register_device_handler`` adds a name (an alias of a kind with fixed
parameters), which is what ``paracel_register_bupdate`` resolves against when
the key lives in a device table.  ``update_file`` is accepted and ignored for
these names: the code is part of the kernel library.

Key filters (``paracel_read_special`` / ``paracel_remove_special``) are
predicates on the key string.  The names shipped with the reference
(alg/recommendation/matrix_factorization/filter.cpp:32-73,
alg/graph_alg/pagerank/update.cpp:40-49) are built in, ``prefix:`` /
``suffix:`` / ``contains:`` forms are parsed, and anything else is looked up
as a Python function exactly like a host filter.
"""
from __future__ import annotations

from typing import Callable, Dict, NamedTuple, Optional

KINDS = ("add", "scaled_add", "sgd", "prox_l1", "max", "assign")
LINEAR_KINDS = ("add", "scaled_add", "sgd")


class DeviceHandler(NamedTuple):
    kind: str
    lr: Optional[float] = None
    lam: Optional[float] = None
    scale: Optional[float] = None


_REG: Dict[str, DeviceHandler] = {k: DeviceHandler(k) for k in KINDS}
for _name in ("default_incr_i", "default_incr_f", "default_incr_d", "default_incr_li",
              "default_incr_lf", "default_incr_ld", "lr_theta_update", "ridge_theta_update",
              "svd_updater", "local_update_kmeans_clusters", "cnt_updater", "mf_fac_updater",
              "mf_bias_updater", "gLDA_topic_update", "gLDA_word_update", "gLDA_sum_topic_update"):
    _REG[_name] = DeviceHandler("add")
_REG["max_updater"] = DeviceHandler("max")


def register_device_handler(name: str, kind: str, lr: Optional[float] = None,
                            lam: Optional[float] = None, scale: Optional[float] = None) -> None:
    """Make ``name`` usable as the ``func_name`` of an update on a device table."""
    if kind not in KINDS:
        raise ValueError(f"unknown device handler kind {kind!r}; choose one of {KINDS}")
    _REG[name] = DeviceHandler(kind, lr, lam, scale)


def resolve_device_handler(name: str) -> DeviceHandler:
    try:
        return _REG[name]
    except KeyError:
        raise KeyError(f"no device handler named {name!r}; known: {sorted(_REG)} "
                       f"(add one with register_device_handler)") from None


def is_device_handler(name: str) -> bool:
    return name in _REG


_FILTERS = {
    "mf_ubias_filter": ("prefix", "usr_bias_"), "mf_ibias_filter": ("prefix", "item_bias_"),
    "mf_W_filter": ("prefix", "W_"), "mf_H_filter": ("prefix", "H_"),
    "mf_cntx_filter": ("suffix", "_u_cnt"), "mf_cnty_filter": ("suffix", "_i_cnt"),
    "pr_filter": ("suffix", "_pr"), "wc_filter": ("prefix", "key_"),
    "gLDA_dump_filter": ("prefix", "key_"),
}


def key_filter(file_name: str, func_name: str) -> Callable[[str], bool]:
    """Predicate on key strings for ``(file_name, func_name)``; an empty name accepts all."""
    if not func_name:
        return lambda key: True
    spec = _FILTERS.get(func_name)
    if spec is None and ":" in func_name:
        how, _, arg = func_name.partition(":")
        if how in ("prefix", "suffix", "contains"):
            spec = (how, arg)
    if spec is not None:
        how, arg = spec
        if how == "prefix":
            return lambda key: key.startswith(arg)
        if how == "suffix":
            return lambda key: key.endswith(arg)
        return lambda key: arg in key
    from .handlers import _load
    fn = _load(file_name, func_name)
    return lambda key: bool(fn(key))
