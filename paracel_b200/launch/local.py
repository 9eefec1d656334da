"""Run a job on one host: P parameter-server daemons plus W worker processes
(the reference's ``local`` mode, prun.py:66-83, 144-176).  Used by the ``prun``
command line and by the tests."""
from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _server_main(q, host: str):
    from ..ps.server import make_server
    srv = make_server()
    port = srv.start(host, 0)
    q.put((host, port))
    srv.wait()
    srv.stop()


def _worker_main(rank: int, world: int, master_port: int, server_info: str, target, args, kwargs,
                 q, backend: str):
    try:
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world)
        os.environ["LOCAL_RANK"] = str(rank)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(master_port)
        os.environ.setdefault("OMP_NUM_THREADS", "1")
        import torch
        torch.set_num_threads(1)
        if "nccl" in backend and torch.cuda.is_available():
            torch.cuda.set_device(rank % torch.cuda.device_count())
        from ..parallel.comm import Comm, main_env
        env = main_env(backend=backend, timeout_s=float(os.environ.get("PCL_PG_TIMEOUT_S", "300")))
        comm = Comm()
        res = target(comm, server_info, *args, **kwargs)
        q.put((rank, "ok", res))
        try:
            comm.synchronize()
        except Exception:
            pass
        env.close()
    except BaseException as e:  # report, never hang the parent
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


class LocalJob:
    """Start servers as child processes, run ``target(comm, server_info, *args)`` in
    ``nworkers`` child processes (gloo ranks), collect the return values."""

    def __init__(self, nworkers: int, nservers: int = 1, backend: str = "gloo"):
        self.nworkers, self.nservers, self.backend = nworkers, nservers, backend
        self.ctx = mp.get_context("spawn")
        self.server_procs: List[Any] = []
        self.endpoints: List[Tuple[str, int]] = []

    def start_servers(self) -> str:
        from ..utils.types import SEPERATOR
        q = self.ctx.Queue()
        for _ in range(self.nservers):
            p = self.ctx.Process(target=_server_main, args=(q, "127.0.0.1"), daemon=True)
            p.start()
            self.server_procs.append(p)
        for _ in range(self.nservers):
            self.endpoints.append(q.get(timeout=120))
        return SEPERATOR.join(f"{h}:{p}" for h, p in self.endpoints)

    def stop_servers(self) -> None:
        from ..ps.client import kvclt
        for (h, p), proc in zip(self.endpoints, self.server_procs):
            try:
                c = kvclt(h, p, timeout_s=5.0)
                c.shutdown()
                c.close()
            except Exception:
                pass
        for proc in self.server_procs:
            proc.join(timeout=5)
            if proc.is_alive():
                proc.terminate()  # SIGTERM first; the reference sends SIGKILL to the group
                proc.join(timeout=5)
            if proc.is_alive():
                proc.kill()
        self.server_procs, self.endpoints = [], []

    def run(self, target: Callable, args: Sequence = (), kwargs: Optional[Dict] = None,
            timeout_s: float = 600.0, server_info: Optional[str] = None) -> List[Any]:
        kwargs = kwargs or {}
        own_servers = server_info is None and self.nservers > 0
        if own_servers:
            server_info = self.start_servers()
        q = self.ctx.Queue()
        port = free_port()
        procs = []
        try:
            for r in range(self.nworkers):
                p = self.ctx.Process(target=_worker_main,
                                     args=(r, self.nworkers, port, server_info, target, tuple(args),
                                           kwargs, q, self.backend))
                p.start()
                procs.append(p)
            results: Dict[int, Any] = {}
            errors: List[str] = []
            import queue as _q
            import time
            deadline = time.time() + timeout_s
            while len(results) + len(errors) < self.nworkers:
                try:
                    rank, status, payload = q.get(timeout=1.0)
                except _q.Empty:
                    if time.time() > deadline:
                        errors.append("timeout waiting for workers")
                        break
                    dead = [i for i, p in enumerate(procs)
                            if not p.is_alive() and p.exitcode not in (0, None) and i not in results]
                    if dead and not errors:
                        # a rank died without reporting: give the others a moment, then stop
                        time.sleep(2.0)
                        errors.append(f"worker(s) {dead} exited abnormally")
                        # drain whatever arrived meanwhile
                        try:
                            while True:
                                rank, status, payload = q.get_nowait()
                                if status == "ok":
                                    results[rank] = payload
                                else:
                                    errors.append(f"rank {rank}: {payload}")
                        except _q.Empty:
                            pass
                        break
                    continue
                if status == "ok":
                    results[rank] = payload
                else:
                    errors.append(f"rank {rank}: {payload}")
                    break
            for p in procs:
                p.join(timeout=10 if not errors else 1)
            for p in procs:
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=5)
            if errors:
                raise RuntimeError("local job failed:\n" + "\n".join(errors))
            return [results[r] for r in range(self.nworkers)]
        finally:
            if own_servers:
                self.stop_servers()
