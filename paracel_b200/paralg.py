"""The ``paralg`` programming interface (reference: include/ps.hpp:67-1342).

A subclass implements ``solve()`` and talks to the parameter servers through
``paracel_read`` / ``paracel_write`` / ``paracel_update`` / ``paracel_bupdate``
and friends, loads its share of the input with ``paracel_load*``, synchronises
with ``paracel_sync`` and, when SSP is switched on, marks the end of an
iteration with ``iter_commit``.  This class is the host-side (CPU) backend:
string keys are placed on servers by the consistent-hash ring and every value
is a msgpack blob.  The GPU backend keeps fixed-width tables in HBM instead
(``paracel_b200.ps.tables``) and is used by the algorithm classes directly.

SSP rule implemented here (intended semantics of ps.hpp:343-355, 401-462):
the first read and the reads after the last iteration always pull; otherwise a
cached value is served while ``stale_cache + limit_s > clock``; else the worker
waits (bounded) until the slowest running worker is at most ``limit_s``
iterations behind, then pulls and refreshes the cache.
"""
from __future__ import annotations

import glob
import heapq
import os
import time
from concurrent.futures import Future
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

from .graph import bigraph, bigraph_continuous, digraph
from .load.loader import loader
from .load.parser import parser_a
from .load.partition import partition
from .parallel.comm import Comm
from .ps.client import kvclt
from .ps.handlers import _load as _load_handler
from .ps.ring import ring
from .utils import dump as _dump
from .utils.decomp import npfact2d, npfactx, npfacty
from .utils.ext import expand, todir
from .utils.misc import get_hostnames_dict
from .utils.packer import pkl_dat_sequential, unpkl_dat_sequential


class ParacelTimeout(RuntimeError):
    """A bounded wait (SSP staleness wait) ran out."""


class parasrv:
    """Connection set to all servers plus the key ring (ps.hpp:1243-1278)."""

    def __init__(self, hosts_dct_str: str, timeout_s: float = 0.0, inproc_servers=None):
        self.kvm: List[kvclt] = []
        if inproc_servers is not None:
            for s in inproc_servers:
                self.kvm.append(kvclt("inproc", 0, inproc=s))
        else:
            for d in get_hostnames_dict(hosts_dct_str):
                port = int(str(d["ports"]).split(",")[0])
                self.kvm.append(kvclt(d["host"], port, timeout_s))
        self.srv_sz = len(self.kvm)
        if self.srv_sz == 0:
            raise ValueError("no parameter server given")
        self.p_ring = ring(range(self.srv_sz))

    def close(self):
        for c in self.kvm:
            c.close()


class paralg:
    def __init__(self, hosts_dct_str: Union[str, Comm, None] = None, comm: Optional[Comm] = None,
                 output: str = "", rounds: int = 1, limit_s: int = 0, ssp_switch: bool = False,
                 inproc_servers=None, wait_timeout_s: float = 60.0):
        if isinstance(hosts_dct_str, Comm):  # paralg(comm, output, rounds): direct usage
            comm, hosts_dct_str = hosts_dct_str, None
        self.worker_comm = comm if comm is not None else Comm()
        self.output = output
        self.nworker = self.worker_comm.get_size()
        self.rounds = rounds
        self.limit_s = int(limit_s)
        self.ssp_switch = bool(ssp_switch)
        self.clock = 0
        self.stale_cache = 0
        self.clock_server = 0
        self.total_iters = rounds
        self.cached_para: Dict[str, Any] = {}
        self.npx, self.npy = 1, 1
        self.wait_timeout_s = wait_timeout_s
        self.update_f: Optional[Callable] = None
        self.ps_obj: Optional[parasrv] = None
        self._init_output(output)
        if hosts_dct_str is not None or inproc_servers is not None:
            self.ps_obj = parasrv(hosts_dct_str or "", inproc_servers=inproc_servers)
            if self.worker_comm.get_rank() == 0:
                self.ps_obj.kvm[self.clock_server].ssp_reset(self.worker_comm.get_size())
            self.paracel_sync()

    def _init_output(self, folder: str) -> None:
        if not folder:
            return
        if self.worker_comm.get_rank() == 0:
            os.makedirs(folder, exist_ok=True)

    def close(self) -> None:
        if self.ps_obj is not None:
            self.ps_obj.close()

    # ------------------------------------------------------------- control
    def iter_commit(self) -> None:
        """End of one iteration under SSP: commit this worker's clock; a worker that has
        finished all its iterations stops being waited for."""
        srv = self.ps_obj.kvm[self.clock_server]
        srv.ssp_commit(self.clock)
        self.clock += 1
        if self.clock == self.total_iters:
            srv.ssp_depart()

    def set_total_iters(self, n: int) -> None:
        self.total_iters = int(n)

    def paracel_sync(self) -> None:
        self.worker_comm.synchronize()

    sync = paracel_sync

    def get_worker_id(self) -> int:
        return self.worker_comm.get_rank()

    def get_worker_size(self) -> int:
        return self.worker_comm.get_size()

    def get_server_size(self) -> int:
        return self.ps_obj.srv_sz

    def get_comm(self) -> Comm:
        return self.worker_comm

    def get_cache(self, key: Optional[str] = None):
        return self.cached_para if key is None else self.cached_para[key]

    def is_cached(self, key: str) -> bool:
        return key in self.cached_para

    def set_decomp_info(self, pattern: str) -> None:
        np_ = self.worker_comm.get_size()
        self.npx, self.npy = npfactx(np_)
        if pattern == "fsmap":
            self.npx, self.npy = npfact2d(np_)
        if pattern == "smap":
            self.npx, self.npy = npfacty(np_)

    def get_decomp_info(self) -> Tuple[int, int]:
        return self.npx, self.npy

    # ------------------------------------------------------------- loading
    def paracel_loadall(self, fn) -> List[str]:
        """Every worker reads every line of the input."""
        names = expand(fn)
        p = partition(names, 1, "linesplit")
        p.files_partition()
        return p.files_load_lines_impl(p.get_start_list()[0], p.get_end_list()[-1])

    def paracel_sequential_loadall(self, fn, func: Callable[[List[str]], None]) -> None:
        """Every worker streams all W blocks of the input, one block at a time."""
        names = expand(fn)
        p = partition(names, self.worker_comm.get_size(), "linesplit")
        p.files_partition()
        for st, en in zip(p.get_start_list(), p.get_end_list()):
            func(p.files_load_lines_impl(st, en))

    def paracel_load(self, fn, parser: Callable = parser_a, pattern: str = "linesplit",
                     mix_flag: bool = False) -> List[str]:
        ld = loader(fn, self.worker_comm, parser, pattern, mix_flag)
        lines = ld.load() if pattern == "linesplit" else ld.fixload()
        self.set_decomp_info(pattern)
        return lines

    def paracel_load_handle(self, fn, func: Callable[[str], None], pattern: str = "linesplit",
                            mix_flag: bool = False) -> None:
        ld = loader(fn, self.worker_comm, parser_a, pattern, mix_flag)
        ld.fixload_handle(func)
        self.set_decomp_info(pattern)

    def paracel_load_as_graph(self, grp, fn, parser: Callable = parser_a, pattern: str = "fmap",
                              mix_flag: bool = False, numeric: bool = True):
        """Fill a ``digraph`` / ``bigraph`` / ``bigraph_continuous`` with this worker's part.
        Returns (rm, cm) for ``bigraph_continuous`` and None otherwise."""
        ld = loader(fn, self.worker_comm, parser, pattern, mix_flag)
        lines = ld.fixload()
        self.paracel_sync()
        maps = ld.create_graph(lines, grp, numeric=numeric)
        self.set_decomp_info(pattern)
        return maps

    def paracel_load_as_matrix(self, fn, parser: Callable = parser_a, pattern: str = "fsmap",
                               mix_flag: bool = False, dense: bool = False, numeric: bool = True):
        """Sparse: (scipy csr block, row map, col map).  Dense (pattern ``fvec``):
        (ndarray, row map)."""
        if pattern == "fvec":
            dense = True
        ld = loader(fn, self.worker_comm, parser, pattern, mix_flag)
        lines = ld.fixload()
        self.paracel_sync()
        out = ld.create_matrix(lines, dense=dense, numeric=numeric)
        self.set_decomp_info(pattern)
        return out

    def paracel_load_as_matrix_device(self, fn, parser: Callable = parser_a, pattern: str = "fsmap",
                                      mix_flag: bool = False, group=None, device=None):
        """Sparse load with numeric ids whose placement, exchange, renumbering and CSR build run
        on the GPUs (``load/device_exchange.py``): every rank parses its share of the lines,
        copies the (row, col, weight) triples to its device, and the triples travel to their
        owners by peer stores.  Returns ``(rowptr int64, col int32, val fp32, rm, cm)`` as device
        tensors; ``rm[i]`` / ``cm[j]`` are the original ids of local row i / column j, exactly the
        maps ``paracel_load_as_matrix`` returns for the same file and pattern."""
        import numpy as np
        import torch
        from .load.device_exchange import DeviceExchange
        ld = loader(fn, self.worker_comm, parser, pattern, mix_flag)
        lines = ld.fixload()
        self.paracel_sync()
        from .load.scheduler import scheduler
        slots = scheduler(self.worker_comm, pattern, mix_flag).lines_organize(lines, parser, numeric=True)
        trip = [t for slot in slots for t in slot]
        dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        a = torch.as_tensor(np.asarray([t[0] for t in trip], dtype=np.int64), device=dev)
        b = torch.as_tensor(np.asarray([t[1] for t in trip], dtype=np.int64), device=dev)
        w = torch.as_tensor(np.asarray([t[2] for t in trip], dtype=np.float32), device=dev)
        ex = DeviceExchange(pattern, group, dev)
        out = ex.load(a, b, w)
        self.set_decomp_info(pattern)
        return out

    # -------------------------------------------------------- registration
    def paracel_register_update(self, file_name: str, func_name: str) -> bool:
        self.update_f = None if not func_name else self._local_handler(file_name, func_name)
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.register_update(file_name, func_name) and ok
        return ok

    def paracel_register_bupdate(self, file_name: str, func_name: str) -> bool:
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.register_bupdate(file_name, func_name) and ok
        return ok

    def paracel_register_read_special(self, file_name: str, func_name: str) -> bool:
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.register_pullall_special(file_name, func_name) and ok
        return ok

    def paracel_register_remove_special(self, file_name: str, func_name: str) -> bool:
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.register_remove_special(file_name, func_name) and ok
        return ok

    # ---------------------------------------------------------------- reads
    def _srv(self, key: str) -> kvclt:
        return self.ps_obj.kvm[self.ps_obj.p_ring.get_server(key)]

    def _ssp_wait(self) -> None:
        t0 = time.time()
        while self.stale_cache + self.limit_s < self.clock:
            self.stale_cache = self.ps_obj.kvm[self.clock_server].pull_int("server_clock")
            if self.stale_cache + self.limit_s >= self.clock:
                break
            if time.time() - t0 > self.wait_timeout_s:
                raise ParacelTimeout(
                    f"worker {self.get_worker_id()}: clock {self.clock} waited "
                    f"{self.wait_timeout_s}s for server_clock >= {self.clock - self.limit_s}, "
                    f"saw {self.stale_cache}")
            time.sleep(0.0005)

    def _ssp_mode(self) -> str:
        if self.clock == 0 or self.clock == self.total_iters:
            return "pull"
        if self.stale_cache + self.limit_s > self.clock:
            return "cache"
        return "wait"

    def paracel_read(self, key: str, default: Any = KeyError) -> Any:
        """Value of ``key``.  A missing key raises KeyError unless ``default`` is given."""
        try:
            if self.ssp_switch:
                mode = self._ssp_mode()
                if mode == "cache" and key in self.cached_para:
                    return self.cached_para[key]
                if mode == "wait":
                    self._ssp_wait()
                val = self._srv(key).pull(key)
                self.cached_para[key] = val
                return val
            return self._srv(key).pull(key)
        except KeyError:
            if default is KeyError:
                raise
            return default

    def _bucket(self, keys: Sequence[str]) -> List[List[str]]:
        lst: List[List[str]] = [[] for _ in range(self.ps_obj.srv_sz)]
        for k in keys:
            lst[self.ps_obj.p_ring.get_server(k)].append(k)
        return lst

    def paracel_read_multi(self, keys: Sequence[str], as_dict: bool = False):
        """List form (values in key order, every key must exist, SSP-aware) or, with
        ``as_dict``, the tolerant form that returns only the keys that exist."""
        keys = list(keys)
        if as_dict:
            out: Dict[str, Any] = {}
            for k, sub in enumerate(self._bucket(keys)):
                if sub:
                    out.update(self.ps_obj.kvm[k].pull_multi_check(sub))
            return out
        if self.ssp_switch:
            mode = self._ssp_mode()
            if mode == "cache" and all(k in self.cached_para for k in keys):
                return [self.cached_para[k] for k in keys]
            if mode == "wait":
                self._ssp_wait()
        vals: Dict[str, Any] = {}
        for k, sub in enumerate(self._bucket(keys)):
            if sub:
                vals.update(zip(sub, self.ps_obj.kvm[k].pull_multi(sub)))
        if self.ssp_switch:
            self.cached_para.update(vals)
        return [vals[k] for k in keys]

    def paracel_readall(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {}
        for c in self.ps_obj.kvm:
            d.update(c.pullall())
        return d

    def paracel_readall_handle(self, func: Callable[[Dict[str, Any]], None]) -> None:
        for c in self.ps_obj.kvm:
            func(c.pullall())

    def paracel_read_special(self, file_name: str = "", func_name: str = "") -> Dict[str, Any]:
        d: Dict[str, Any] = {}
        for c in self.ps_obj.kvm:
            d.update(c.pullall_special(file_name, func_name))
        return d

    def paracel_read_special_handle(self, file_name: str, func_name: str,
                                    func: Callable[[Dict[str, Any]], None]) -> None:
        for c in self.ps_obj.kvm:
            func(c.pullall_special(file_name, func_name))

    @staticmethod
    def _topk(k: int, feed: Callable[[Callable], None]) -> List[Tuple[str, Any]]:
        heap: List[Tuple[Any, str]] = []

        def handler(d: Dict[str, Any]):
            for key, v in d.items():
                if len(heap) < k:
                    heapq.heappush(heap, (v, key))
                elif v > heap[0][0]:
                    heapq.heapreplace(heap, (v, key))
        feed(handler)
        return [(key, v) for v, key in sorted(heap, reverse=True)]

    def paracel_read_topk(self, k: int) -> List[Tuple[str, Any]]:
        """The k largest values over all servers as (key, value), largest first (all
        parameters must be of one comparable type)."""
        return self._topk(k, self.paracel_readall_handle)

    def paracel_read_topk_with_key_filter(self, k: int, file_name: str, func_name: str):
        return self._topk(k, lambda h: self.paracel_read_special_handle(file_name, func_name, h))

    # --------------------------------------------------------------- writes
    def paracel_write(self, key: str, val: Any, replica_flag: bool = False) -> bool:
        if self.ssp_switch:
            self.cached_para[key] = val
        return self._srv(key).push(key, val)

    def paracel_write_multi(self, dct: Dict[str, Any]) -> bool:
        buckets: List[Dict[str, Any]] = [dict() for _ in range(self.ps_obj.srv_sz)]
        for k, v in dct.items():
            if self.ssp_switch:
                self.cached_para[k] = v
            buckets[self.ps_obj.p_ring.get_server(k)][k] = v
        ok = True
        for i, b in enumerate(buckets):
            if b:
                ok = self.ps_obj.kvm[i].push_multi(b) and ok
        return ok

    def _local_handler(self, file_name: str, func_name: str) -> Callable:
        from ._core import core
        from .utils.packer import pack, unpack
        if core().handler_is_builtin(func_name):
            return lambda a, b: unpack(core().apply_builtin_handler(func_name, pack(a), pack(b)))
        return _load_handler(file_name, func_name)

    def paracel_update(self, key: str, delta: Any, file_name: str = "", func_name: str = "") -> Future:
        """Non-blocking update; returns a future.  Under SSP the handler is also applied
        to the locally cached copy (ps.hpp:689-750)."""
        if self.ssp_switch and key in self.cached_para:
            f = self._local_handler(file_name, func_name) if func_name else self.update_f
            if f is None:
                f = self._local_handler("", "default_incr_d")
            self.cached_para[key] = f(self.cached_para[key], delta)
        return self._srv(key).update(key, delta, file_name, func_name)

    def paracel_bupdate(self, key: str, delta: Any, file_name: str = "", func_name: str = "") -> bool:
        """Blocking update; under SSP the cache takes the server's new value."""
        new_val = self._srv(key).bupdate(key, delta, file_name, func_name)
        if self.ssp_switch:
            self.cached_para[key] = new_val
        return True

    def paracel_bupdate_multi(self, keys, deltas=None, file_name: str = "", func_name: str = "") -> bool:
        """``(keys, deltas, file, func)`` or ``(dict, file, func)``."""
        if isinstance(keys, dict):
            if deltas is not None and not isinstance(deltas, (list, tuple)):
                file_name, func_name = deltas, file_name  # (dict, file, func) call shape
            items = list(keys.items())
        else:
            items = list(zip(keys, deltas))
        buckets: List[Tuple[List[str], List[Any]]] = [([], []) for _ in range(self.ps_obj.srv_sz)]
        for k, d in items:
            b = buckets[self.ps_obj.p_ring.get_server(k)]
            b[0].append(k)
            b[1].append(d)
        for i, (ks, ds) in enumerate(buckets):
            if ks:
                new_vals = self.ps_obj.kvm[i].bupdate_multi(ks, ds, file_name, func_name)
                if self.ssp_switch:
                    self.cached_para.update(zip(ks, new_vals))
        return True

    def paracel_contains(self, key: str) -> bool:
        return self._srv(key).contains(key)

    def paracel_remove(self, key: str) -> bool:
        self.cached_para.pop(key, None)
        return self._srv(key).remove(key)

    def paracel_remove_multi(self, keys: Sequence[str]) -> bool:
        """Remove several keys (a stub in the reference, ps.hpp:920-927)."""
        ok = True
        for k in keys:
            ok = self.paracel_remove(k) and ok
        return ok

    def paracel_remove_special(self, file_name: str = "", func_name: str = "") -> bool:
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.remove_special(file_name, func_name) and ok
        return ok

    def data_merge(self, data: Any, func: Callable[[Any, Any], Any], comm: Optional[Comm] = None,
                   rank: int = 0) -> Any:
        return (comm or self.worker_comm).treereduce(data, func, rank)

    # ---------------------------------------------------- persistence / dump
    def pkl_dat(self, data: Any, prefix: str = "result_") -> None:
        path = todir(self.output) + prefix + str(self.get_worker_id()) + ".pkl"
        pkl_dat_sequential(data, path)

    def unpkl_dat(self, prefix: str = "result_", cols: int = 0, sparse: bool = False) -> Any:
        """Read back what :meth:`pkl_dat` wrote (an empty TODO in the reference, ps.hpp:940)."""
        path = todir(self.output) + prefix + str(self.get_worker_id()) + ".pkl"
        return unpkl_dat_sequential(path, cols=cols, sparse=sparse)

    def _dump_path(self, filename: str) -> str:
        return todir(self.output) + filename + str(self.get_worker_id())

    def files_merge(self, filename: str) -> None:
        _dump.files_merge(todir(self.output) + filename + "*", todir(self.output) + filename + "merge")

    def _maybe_merge(self, filename: str, merge: bool) -> None:
        if merge:
            self.paracel_sync()
            if self.get_worker_id() == 0:
                self.files_merge(filename)

    def paracel_dump_vector(self, data: Sequence, filename: str = "result_", sep: str = ",",
                            append_flag: bool = False, merge: bool = False) -> None:
        _dump.dump_vector(data, self._dump_path(filename), sep, append_flag)
        self._maybe_merge(filename, merge)

    def paracel_dump_dict(self, data: Dict, filename: str = "result_", append_flag: bool = False,
                          merge: bool = False) -> None:
        """Chooses the line layout from the value type: scalar -> ``key\\tvalue``; list of
        numbers -> ``key\\tv0|v1|...``; list of (key, number) pairs -> ``key\\tk0:v0|k1:v1``."""
        path = self._dump_path(filename)
        sample = next(iter(data.values()), None)
        if isinstance(sample, (list, tuple)):
            first = sample[0] if len(sample) else None
            if isinstance(first, (list, tuple)) and len(first) == 2:
                _dump.dump_dict_pairs(data, path, append_flag)
            else:
                _dump.dump_dict_vector(data, path, append_flag)
        else:
            _dump.dump_dict_scalar(data, path, append_flag)
        self._maybe_merge(filename, merge)

    def paracel_dump_prob_mtx(self, data: Dict, filename: str = "result_", append_flag: bool = False,
                              merge: bool = False) -> None:
        _dump.dump_prob_mtx(data, self._dump_path(filename), append_flag)
        self._maybe_merge(filename, merge)

    def solve(self) -> None:  # pragma: no cover - overridden by algorithms
        pass
