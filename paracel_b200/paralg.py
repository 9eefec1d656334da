"""The ``paralg`` programming interface (reference: include/ps.hpp:67-1342).

A subclass implements ``solve()`` and talks to the parameter servers through
``paracel_read`` / ``paracel_write`` / ``paracel_update`` / ``paracel_bupdate``
and friends, loads its share of the input with ``paracel_load*``, synchronises
with ``paracel_sync`` and, when SSP is switched on, marks the end of an
iteration with ``iter_commit``.

Two backends sit behind the same calls.  The host backend places string keys on
server processes by the consistent-hash ring; every value is a msgpack blob.
With ``backend="gpu"`` the object also owns a directory of typed tables whose
shards live in the HBM of the ranks (``paracel_b200.ps.device_store``): keys
that match a registered table -- ``"theta"``, ``"W_<id>"``, ``"<id>_pr"`` --
are served by kernels that read, reduce into and store to the owners' memory
over NVLink, with the handler named in ``paracel_bupdate`` applied at the owner
and the SSP clock kept in device memory; all other keys go to the host servers
as before.  Bulk calls take a ``KeyBatch`` (an id tensor plus the key pattern)
and device tensors, so no per-key loop runs on the training path.

SSP rule implemented here (intended semantics of ps.hpp:343-355, 401-462):
the first read and the reads after the last iteration always pull; otherwise a
cached value is served while ``stale_cache + limit_s > clock``; else the worker
waits (bounded) until the slowest running worker is at most ``limit_s``
iterations behind, then pulls and refreshes the cache.
"""
from __future__ import annotations

import heapq
import os
import time
from concurrent.futures import Future
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

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


class _NullPhase:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL_PHASE = _NullPhase()


class _DeviceFuture:
    """Handle of an update queued on a CUDA stream (the device form of the ``std::future`` that
    the reference's ``paracel_update`` returns, include/ps.hpp:689-710)."""

    def __init__(self, event):
        self._event = event

    def done(self) -> bool:
        return self._event.query()

    def result(self, timeout=None) -> bool:
        self._event.synchronize()
        return True


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
                 inproc_servers=None, wait_timeout_s: float = 60.0, backend: str = "cpu",
                 device=None, group=None):
        if isinstance(hosts_dct_str, Comm):  # paralg(comm, output, rounds): direct usage
            comm, hosts_dct_str = hosts_dct_str, None
        self.worker_comm = comm if comm is not None else Comm(group)
        if backend not in ("cpu", "gpu"):
            raise ValueError("backend must be 'cpu' or 'gpu'")
        self.backend = backend
        self.dev = None            # DeviceStore: directory + tables in HBM (gpu backend)
        self.dev_clock = None      # DeviceSspClock
        self._dev_pulled_at: Dict[Any, int] = {}
        self._dev_default_bupdate = ""
        self._dev_waited = None
        self.metrics = None        # MetricsLogger, see paracel_enable_metrics
        self.timer = None          # PhaseTimer
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
        if backend == "gpu":
            from .parallel.ssp_device import DeviceSspClock
            from .ps.device_store import DeviceStore
            grp = group if group is not None else self.worker_comm.group
            self.dev = DeviceStore(grp, device)
            self.device = self.dev.device
            self.dev_clock = DeviceSspClock(self.limit_s if self.ssp_switch else 0, self.rounds,
                                            grp, self.device, min(wait_timeout_s, 30.0))

    def _init_output(self, folder: str) -> None:
        if not folder:
            return
        if self.worker_comm.get_rank() == 0:
            os.makedirs(folder, exist_ok=True)

    def close(self) -> None:
        if self.metrics is not None:
            self.metrics.close()
            self.metrics = None
        if self.ps_obj is not None:
            self.ps_obj.close()
            self.ps_obj = None
        if self.dev is not None:
            self.paracel_sync()
            self.dev.free()
            self.dev_clock.free()
            self.dev = self.dev_clock = None

    # ------------------------------------------------- device tables (gpu backend)
    def _need_dev(self):
        if self.dev is None:
            raise RuntimeError("this paralg object was built with backend='cpu'; device tables "
                               "need backend='gpu'")
        return self.dev

    def paracel_dense_table(self, key: str, length: int, handler: str = "add", lr: float = 1.0,
                            lam: float = 0.0):
        """Register ``key`` as a dense fp32 vector of ``length`` elements range-sharded over the
        ranks' HBM (collective).  ``handler`` is the default of ``paracel_bupdate`` on the key."""
        return self._need_dev().add_dense(key, length, handler, lr, lam,
                                          timeout_s=min(self.wait_timeout_s, 30.0))

    def paracel_row_table(self, rows: int, width: int, prefix: str = "", suffix: str = "",
                          dtype=None, names=None, handler: str = "add"):
        """Register the keys ``prefix<id>suffix`` as fixed-width rows (fp32 or int32) sharded by
        ``row % world`` (collective).  ``names``: sorted original ids, row r <-> names[r]."""
        import torch
        return self._need_dev().add_rows(rows, width, prefix, suffix,
                                         torch.float32 if dtype is None else dtype, names, handler)

    def paracel_scalar_table(self, rows: int, prefix: str = "", suffix: str = "", names=None,
                             handler: str = "add"):
        return self._need_dev().add_scalars(rows, prefix, suffix, names, handler)

    def paracel_matrix_table(self, key: str, rows: int, cols: int, kernel=None):
        """Register ``key`` as a row-sharded matrix that is read through the fused all-gather +
        tcgen05 GEMM (``paracel_read_matmul``)."""
        return self._need_dev().add_matrix(key, rows, cols, kernel)

    def paracel_keys(self, table, ids, original_ids: bool = False):
        """The key batch ``prefix<id>suffix`` of ``table`` for a tensor of rows (or, with
        ``original_ids``, of ids of the input file)."""
        return self._need_dev().batch(table, ids, original_ids)

    def paracel_local_shard(self, key_or_table):
        """This rank's shard of a device table, as a tensor in its own HBM (owner-side access:
        an owner may initialise or rewrite its part in place, then ``paracel_commit_write``)."""
        e = key_or_table if not isinstance(key_or_table, str) else self._need_dev()._exact[key_or_table]
        return e.table.shard

    def paracel_commit_write(self, key_or_table) -> None:
        """Publish an in-place rewrite of this rank's shard of a dense key: the next read of the
        key on any rank waits until every owner has published."""
        e = key_or_table if not isinstance(key_or_table, str) else self._need_dev()._exact[key_or_table]
        e.table.mark_written()

    def paracel_read_matmul(self, key: str, A, out=None, argmin_bnorm=None):
        """``A @ value(key).T`` (or its row-wise arg-min with ``argmin_bnorm``) with the read of
        the matrix key fused into the GEMM."""
        e = self._need_dev()._exact[key]
        return e.table.g(A, out, argmin_bnorm)

    def _dev_hit(self, key):
        if self.dev is None or not isinstance(key, str):
            return None
        return self.dev.resolve(key)

    def _dev_ssp_target(self, cache_key, peek: bool = False) -> Optional[int]:
        """SSP rule for a device read: None = serve the caller's cached copy, else the minimum
        clock the pull has to wait for (0 = no wait).  A copy pulled at clock c is served while
        ``clock - c < limit_s``; the first read and the reads after the last iteration pull."""
        if not self.ssp_switch:
            return 0
        if self.limit_s > 0:
            at = self._dev_pulled_at.get(cache_key)
            if at is not None and 0 < self.clock < self.total_iters and self.clock - at < self.limit_s:
                return None
            if not peek:
                self._dev_pulled_at[cache_key] = self.clock
        return max(0, self.clock - self.limit_s)

    @staticmethod
    def _dev_cache_key(kb, out):
        return ("b", id(kb.entry), 0 if out is None else out.data_ptr())

    def paracel_would_pull(self, keys, out=None) -> bool:
        """Whether ``paracel_read_multi(keys, out=out)`` would transfer rows now (True) or serve
        the copy already in ``out`` under the SSP cache rule (False)."""
        return self._dev_ssp_target(self._dev_cache_key(keys, out), peek=True) is not None

    def paracel_invalidate_cache(self) -> None:
        """Forget which device copies are fresh: the next read of every key pulls."""
        self._dev_pulled_at.clear()

    def _dev_wait_needed(self, target: int) -> bool:
        """True once per (clock, stream): whether a staleness wait for ``target`` still has to be
        queued on the current stream (reads of several tables in one iteration share one wait)."""
        if target <= 0 or self.dev is None or self.dev.world == 1:
            return False
        from .ops import _lib
        mark = (self.clock, _lib.stream_ptr())
        if self._dev_waited == mark:
            return False
        self._dev_waited = mark
        return True

    def _host(self, key=None) -> parasrv:
        if self.ps_obj is None:
            raise KeyError(f"key {key!r} matches no device table and no host parameter server "
                           f"is connected")
        return self.ps_obj

    # ------------------------------------------- checkpoint / resume, metrics, phases
    def checkpoint_extra(self) -> Dict[str, Any]:
        """Model state beyond the tables that a checkpoint has to carry (tensors / plain values);
        subclasses override together with :meth:`restore_extra`."""
        return {}

    def restore_extra(self, extra: Dict[str, Any]) -> None:
        pass

    def save_checkpoint(self, ckpt_dir: str) -> None:
        """Collective.  Writes, per rank, this rank's shard of every device table, the SSP clock
        and the model's extra state (``rank<r>.pt``); rank 0 adds ``meta.json`` and, when host
        servers are connected, their shards (``servers.pkl``).  Files are written under a
        temporary name and renamed."""
        from .utils import checkpoint as ck
        self.paracel_sync()
        state: Dict[str, Any] = {"clock": self.clock, "extra": self.checkpoint_extra()}
        if self.dev is not None:
            for j, e in enumerate(self.dev.entries):
                state[f"table{j}"] = {"pattern": e.pattern, "kind": e.kind, "shard": e.table.shard}
        ck.save_rank_state(ckpt_dir, self.get_worker_id(), state)
        if self.ps_obj is not None:
            ck.save_servers(self, ckpt_dir)
        self.paracel_sync()
        if self.get_worker_id() == 0:
            ck.save_meta(ckpt_dir, {"world": self.get_worker_size(), "clock": self.clock,
                                    "total_iters": self.total_iters, "class": type(self).__name__})
        self.paracel_sync()

    def load_checkpoint(self, ckpt_dir: str) -> None:
        """Collective.  Restores what :meth:`save_checkpoint` wrote into an object that was built
        and loaded the same way (same tables, same world size, same data): table shards, SSP clock
        (device clock words included), the model's extra state.  Cached copies are dropped."""
        from .utils import checkpoint as ck
        meta = ck.load_meta(ckpt_dir)
        if meta["world"] != self.get_worker_size():
            raise ValueError(f"checkpoint of {meta['world']} workers loaded by {self.get_worker_size()}")
        state = ck.load_rank_state(ckpt_dir, self.get_worker_id())
        self.paracel_sync()
        if self.dev is not None:
            for j, e in enumerate(self.dev.entries):
                rec = state.get(f"table{j}")
                if rec is None or rec["pattern"] != e.pattern or rec["kind"] != e.kind:
                    raise ValueError(f"checkpoint has no table {e.pattern!r} at position {j}")
                e.table.shard.copy_(rec["shard"].to(self.device).view_as(e.table.shard))
        if self.ps_obj is not None and os.path.exists(os.path.join(ckpt_dir, "servers.pkl")):
            ck.load_servers(self, ckpt_dir)
        self.clock = int(state["clock"])
        if self.dev_clock is not None:
            self.dev_clock.restore(self.clock)
        self.cached_para.clear()
        self.paracel_invalidate_cache()
        self.restore_extra(state.get("extra", {}))
        self.paracel_sync()

    def paracel_enable_metrics(self, path: Optional[str] = None, phases: bool = True, nvtx: bool = False,
                               only_rank0: bool = True) -> None:
        """Switch on ``metrics.jsonl`` (one JSON object per ``log_metrics`` call; default path
        ``<output>/metrics.jsonl``) and per-phase timing with CUDA events (``phase`` blocks;
        NVTX ranges with ``nvtx``).  Both are off by default and cost nothing then."""
        from .utils.metrics import MetricsLogger, PhaseTimer
        if path is None:
            path = todir(self.output or ".") + "metrics.jsonl"
        self.metrics = MetricsLogger(path, self.get_worker_id(), only_rank0)
        self.timer = PhaseTimer(nvtx=nvtx) if phases else None

    def log_metrics(self, **kv: Any) -> None:
        if self.metrics is not None:
            kv.setdefault("clock", self.clock)
            self.metrics.log(**kv)

    def phase(self, name: str):
        """Context manager that times a named phase on the current stream when phase timing is on."""
        if self.timer is None:
            return _NULL_PHASE
        return self.timer.phase(name)

    def phase_summary(self) -> Dict[str, Dict[str, float]]:
        """{phase: {ms, count}} since the last call (synchronises the device once)."""
        return self.timer.summary() if self.timer is not None else {}

    def dump_phase_trace(self, path: Optional[str] = None) -> None:
        """Write this rank's phase totals to ``<output>/trace_rank<r>.json``."""
        if self.timer is not None:
            self.timer.dump(path or (todir(self.output or ".") + f"trace_rank{self.get_worker_id()}.json"),
                            self.get_worker_id())

    # ------------------------------------------------------------- control
    def iter_commit(self) -> None:
        """End of one iteration under SSP: commit this worker's clock; a worker that has
        finished all its iterations stops being waited for.  With device tables the clock word
        is stored into every peer's HBM by one small kernel, ordered after this worker's
        earlier pushes."""
        if self.dev_clock is not None:
            self.dev_clock.commit()
        if self.ps_obj is not None:
            srv = self.ps_obj.kvm[self.clock_server]
            srv.ssp_commit(self.clock)
        self.clock += 1
        if self.clock == self.total_iters and self.ps_obj is not None:
            self.ps_obj.kvm[self.clock_server].ssp_depart()

    def set_total_iters(self, n: int) -> None:
        self.total_iters = int(n)
        if self.dev_clock is not None:
            self.dev_clock.total_iters = int(n)

    def paracel_sync(self) -> None:
        if self.dev is not None:
            import torch
            torch.cuda.synchronize(self.device)
        self.worker_comm.synchronize()

    def paracel_check(self) -> None:
        """Raise what the device side reported since the last check: a staleness or table wait
        that ran out (``SspTimeout`` / ``DeviceWaitTimeout``) or an id outside its table
        (``BadDeviceId``).  Synchronises the device; the tables must be treated as undefined
        after a timeout (pushes and commits of the failed round were skipped)."""
        if self.dev is not None:
            self.dev_clock.check()
            self.dev.check()

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
        if self.dev is not None and self.ps_obj is None:
            from .ps.device_handlers import resolve_device_handler
            resolve_device_handler(func_name)
            self._dev_default_bupdate = func_name
            return True
        self.update_f = None if not func_name else self._local_handler(file_name, func_name)
        ok = True
        for c in self.ps_obj.kvm:
            ok = c.register_update(file_name, func_name) and ok
        return ok

    def paracel_register_bupdate(self, file_name: str, func_name: str) -> bool:
        ok = True
        if self.dev is not None:
            from .ps.device_handlers import is_device_handler
            if is_device_handler(func_name):
                self._dev_default_bupdate = func_name
            elif self.ps_obj is None:
                raise KeyError(f"no device handler named {func_name!r}")
        if self.ps_obj is not None:
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
        ps = self._host(key)
        return ps.kvm[ps.p_ring.get_server(key)]

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
        """Value of ``key``.  A missing key raises KeyError unless ``default`` is given.  A key
        of a device table returns a device tensor (dense vector, row) or a float (scalar)."""
        hit = self._dev_hit(key)
        if hit is not None:
            e, row = hit
            if e.kind == "dense":
                tgt = self._dev_ssp_target(("k", key))
                if tgt is None:
                    if self._dev_wait_needed(self.clock - self.limit_s):
                        self.dev_clock.wait()
                    return e.table.full[: e.table.L]
                if self._dev_wait_needed(tgt):
                    self.dev_clock.wait()
            return self.dev.read_key(e, row)
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

    def paracel_read_multi(self, keys, as_dict: bool = False, out=None, snapshot=None,
                           ssp_wait: bool = True, use_cache: bool = True):
        """List form (values in key order, every key must exist, SSP-aware) or, with
        ``as_dict``, the tolerant form that returns only the keys that exist.

        Device form: ``keys`` is a ``KeyBatch``; the rows are gathered from their owners' HBM by
        one kernel into ``out`` (allocated if missing; ``snapshot`` receives a second copy, the
        "old" value of a later delta push) and ``out`` is returned.  Under SSP the kernel first
        waits, bounded, until no worker is more than ``limit_s`` clocks behind; while the copy
        in ``out`` is younger than ``limit_s`` clocks it is served as it is.  ``ssp_wait=False``
        reads without the staleness wait (evaluation outside the training loop);
        ``use_cache=False`` always transfers (callers that reuse one buffer for changing keys)."""
        from .ps.device_store import KeyBatch
        if isinstance(keys, KeyBatch):
            if use_cache:
                tgt = self._dev_ssp_target(self._dev_cache_key(keys, out))
            else:
                tgt = max(0, self.clock - self.limit_s) if self.ssp_switch else 0
            if tgt is None and out is not None:
                # the staleness bound holds for cached copies too
                if ssp_wait and self._dev_wait_needed(self.clock - self.limit_s):
                    self.dev_clock.wait()
                return out
            clk = self.dev_clock if (ssp_wait and self._dev_wait_needed(tgt or 0)) else None
            return self.dev.pull(keys, out, snapshot, clk, tgt or 0)
        keys = list(keys)
        if self.dev is not None and keys:
            groups, host_pos = self.dev.group_keys(keys)
            if groups:
                vals: List[Any] = [None] * len(keys)
                for e, pos, kb in groups:
                    got = self.dev.pull(kb)
                    rows = got.cpu().tolist() if e.kind == "scalars" else list(got.unbind(0))
                    for p_, v in zip(pos, rows):
                        vals[p_] = v
                if host_pos:
                    hv = self.paracel_read_multi([keys[p_] for p_ in host_pos], as_dict)
                    if as_dict:
                        hv = [hv.get(keys[p_]) for p_ in host_pos]
                    for p_, v in zip(host_pos, hv):
                        vals[p_] = v
                if as_dict:
                    return {k: v for k, v in zip(keys, vals) if v is not None}
                return vals
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

    def _dev_tables_as_dicts(self, file_name: str = "", func_name: str = ""):
        """One ``{key: value}`` dict per device table whose keys pass the filter (rows as lists)."""
        if self.dev is None:
            return
        for e in self.dev.matching(file_name, func_name):
            yield self.dev.dump_entry(e)

    def paracel_readall(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {}
        if self.ps_obj is not None:
            for c in self.ps_obj.kvm:
                d.update(c.pullall())
        for part in self._dev_tables_as_dicts():
            d.update(part)
        return d

    def paracel_readall_handle(self, func: Callable[[Dict[str, Any]], None]) -> None:
        if self.ps_obj is not None:
            for c in self.ps_obj.kvm:
                func(c.pullall())
        for part in self._dev_tables_as_dicts():
            func(part)

    def paracel_read_special(self, file_name: str = "", func_name: str = "") -> Dict[str, Any]:
        """Every parameter whose key passes the filter: host shards and device tables alike (a
        device table is selected as a whole by the filter's answer for its key pattern)."""
        d: Dict[str, Any] = {}
        if self.ps_obj is not None:
            for c in self.ps_obj.kvm:
                d.update(c.pullall_special(file_name, func_name))
        for part in self._dev_tables_as_dicts(file_name, func_name):
            d.update(part)
        return d

    def paracel_read_special_handle(self, file_name: str, func_name: str,
                                    func: Callable[[Dict[str, Any]], None]) -> None:
        if self.ps_obj is not None:
            for c in self.ps_obj.kvm:
                func(c.pullall_special(file_name, func_name))
        for part in self._dev_tables_as_dicts(file_name, func_name):
            func(part)

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
        """Store ``val`` under ``key``.  Device tables: a row or scalar is stored into its owner's
        HBM by this rank alone; a dense key is written collectively (every rank passes the same
        vector, each owner keeps its slice and the next read waits for all owners).  Other
        ranks see a one-sided write after the next ``paracel_sync`` or clock commit."""
        hit = self._dev_hit(key)
        if hit is not None:
            self.dev.write_key(hit[0], hit[1], val)
            return True
        if self.ssp_switch:
            self.cached_para[key] = val
        return self._srv(key).push(key, val)

    def paracel_write_multi(self, dct, values=None) -> bool:
        """``{key: value}``, or the device form ``(KeyBatch, values tensor)``: one kernel stores
        the rows into their owners' HBM."""
        from .ps.device_store import KeyBatch
        if isinstance(dct, KeyBatch):
            self.dev.push(dct, values, "assign")
            return True
        if self.dev is not None and dct:
            keys = list(dct.keys())
            groups, host_pos = self.dev.group_keys(keys)
            for e, pos, kb in groups:
                import torch
                t = e.table
                if e.kind == "scalars":
                    v = torch.tensor([float(dct[keys[p_]]) for p_ in pos], device=self.device)
                else:
                    v = torch.zeros(len(pos), t.width, dtype=t.dtype, device=self.device)
                    for j, p_ in enumerate(pos):
                        row = torch.as_tensor(dct[keys[p_]], dtype=t.dtype)
                        v[j, : row.numel()] = row.to(self.device)
                self.dev.push(kb, v, "assign")
            if not host_pos:
                return True
            dct = {keys[p_]: dct[keys[p_]] for p_ in host_pos}
        self._host(next(iter(dct), None))
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

    def _dev_update(self, hit, delta, func_name: str, collective: Optional[bool],
                    lr: Optional[float] = None, lam: Optional[float] = None):
        """Update of one device key with a named handler (see paracel_bupdate)."""
        import torch
        from .ps.device_handlers import LINEAR_KINDS, resolve_device_handler
        e, row = hit
        name = func_name or self._dev_default_bupdate or e.handler
        h = resolve_device_handler(name)
        if e.kind == "dense":
            t = e.table
            d = torch.as_tensor(delta, dtype=torch.float32, device=self.device)
            if collective is None:
                collective = h.kind not in LINEAR_KINDS
            if collective:
                buf = t.delta()
                if d.data_ptr() != buf.data_ptr():
                    buf.copy_(d)
                t.bupdate(handler=name, lr=lr, lam=lam)
            else:
                if h.kind not in LINEAR_KINDS:
                    raise ValueError(f"handler {name!r} ({h.kind}) is not linear: it needs the "
                                     f"collective form (every worker calls it once per round)")
                scale = 1.0
                if h.kind == "scaled_add":
                    scale = 1.0 if h.scale is None else h.scale
                elif h.kind == "sgd":
                    scale = -(lr if lr is not None else (t.lr if h.lr is None else h.lr))
                t.push(d.contiguous(), scale)
            return
        if e.kind == "matrix":
            raise TypeError(f"{e.key!r} is a matrix table: owners rewrite their shard")
        t = e.table
        v = torch.as_tensor(delta, dtype=t.dtype, device=self.device).reshape(1, -1)
        if e.kind == "rows" and v.shape[1] != t.width:
            full = torch.zeros(1, t.width, dtype=t.dtype, device=self.device)
            full[:, : v.shape[1]] = v
            v = full
        self.dev.push(self.dev.batch(e, [row]), v.reshape(-1) if e.kind == "scalars" else v.contiguous(),
                      name)

    def paracel_update(self, key: str, delta: Any, file_name: str = "", func_name: str = "",
                       collective: Optional[bool] = False) -> Future:
        """Non-blocking update; returns a future.  Under SSP the handler is also applied
        to the locally cached copy (ps.hpp:689-750).  On a device table the update is a
        one-sided reduction into the owner's HBM queued on the current stream; the future
        completes when the kernel has run."""
        hit = self._dev_hit(key)
        if hit is not None:
            import torch
            self._dev_update(hit, delta, func_name, collective)
            ev = torch.cuda.Event()
            ev.record()
            return _DeviceFuture(ev)
        if self.ssp_switch and key in self.cached_para:
            f = self._local_handler(file_name, func_name) if func_name else self.update_f
            if f is None:
                f = self._local_handler("", "default_incr_d")
            self.cached_para[key] = f(self.cached_para[key], delta)
        return self._srv(key).update(key, delta, file_name, func_name)

    def paracel_bupdate(self, key: str, delta: Any, file_name: str = "", func_name: str = "",
                        collective: Optional[bool] = None, lr: Optional[float] = None,
                        lam: Optional[float] = None) -> bool:
        """Blocking update; under SSP the cache takes the server's new value.

        Device tables: ``func_name`` selects the handler that the kernel applies at the owner
        (``paracel_b200.ps.device_handlers``).  A dense key has two forms.  One-sided (default
        for the linear handlers add / scaled add / sgd): this worker alone reduces its delta
        into the owners' shards, whenever and as often as it likes, like the reference's RPC.
        Collective (``collective=True``; the only form of the non-linear handlers prox-L1 and
        max): every worker calls once per round, and each owner sums its slice of all workers'
        deltas out of peer memory and applies the handler in the same kernel -- the
        reduce-scatter fused with the update.  Writing the delta into
        ``paracel_delta_buffer(key)`` saves the copy.  ``lr`` / ``lam`` set the step and the
        threshold of the sgd and prox-L1 handlers for this call (the reference compiles such
        constants into the handler's shared object)."""
        hit = self._dev_hit(key)
        if hit is not None:
            self._dev_update(hit, delta, func_name, collective, lr, lam)
            return True
        new_val = self._srv(key).bupdate(key, delta, file_name, func_name)
        if self.ssp_switch:
            self.cached_para[key] = new_val
        return True

    def paracel_delta_buffer(self, key: str):
        """The buffer (device tensor, full length) that the next collective ``paracel_bupdate``
        of a dense key reduces: a gradient kernel may write its result straight into it."""
        return self._need_dev()._exact[key].table.delta()

    def paracel_bupdate_multi(self, keys, deltas=None, file_name: str = "", func_name: str = "",
                              old=None, wgt=None, refresh_old: bool = True, start: int = 0) -> bool:
        """``(keys, deltas, file, func)`` or ``(dict, file, func)``; device form
        ``(KeyBatch, values, file, func, old=, wgt=, start=)``: one kernel reduces
        ``wgt * (values - old)`` (``values`` itself without ``old``) into the owners' rows with
        the named handler and then refreshes ``old``."""
        from .ps.device_store import KeyBatch
        if isinstance(keys, KeyBatch):
            self.dev.push(keys, deltas, func_name or self._dev_default_bupdate or None, old, wgt,
                          refresh_old, start, self.dev_clock.status if self.dev_clock else None)
            return True
        if isinstance(keys, dict):
            if deltas is not None and not isinstance(deltas, (list, tuple)):
                file_name, func_name = deltas, file_name  # (dict, file, func) call shape
            items = list(keys.items())
        else:
            items = list(zip(keys, deltas))
        if self.dev is not None and items:
            import torch
            ks = [k for k, _ in items]
            groups, host_pos = self.dev.group_keys(ks)
            for e, pos, kb in groups:
                t = e.table
                if e.kind == "scalars":
                    v = torch.tensor([float(items[p_][1]) for p_ in pos], device=self.device)
                else:
                    v = torch.zeros(len(pos), t.width, dtype=t.dtype, device=self.device)
                    for j, p_ in enumerate(pos):
                        row = torch.as_tensor(items[p_][1], dtype=t.dtype)
                        v[j, : row.numel()] = row.to(self.device)
                self.dev.push(kb, v, func_name or self._dev_default_bupdate or None)
            if not host_pos:
                return True
            items = [items[p_] for p_ in host_pos]
        self._host(items[0][0] if items else None)
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
        if self._dev_hit(key) is not None:
            return True            # every row of a registered table exists (zero until written)
        if self.dev is not None and self.ps_obj is None:
            return False
        return self._srv(key).contains(key)

    def paracel_remove(self, key: str) -> bool:
        hit = self._dev_hit(key)
        if hit is not None:
            e, row = hit
            if e.kind in ("dense", "matrix"):
                self.dev.drop(e)           # collective: the table is freed
            else:                          # a row cannot leave its table: it reads as zero again
                self.dev.write_key(e, row, [0] * e.table.width)
            return True
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
