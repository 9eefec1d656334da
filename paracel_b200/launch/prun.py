"""Job launcher with the reference's command line (prun.py:86-176):

    python -m paracel_b200.launch.prun -w 2 -p 1 -c cfg.json -m local lr
    python -m paracel_b200.launch.prun -w 4 -p 2 -c cfg.json -m local ./my_driver --extra flag

It starts ``-p`` parameter-server daemons, collects their ``host:port`` through a rendezvous
socket (the reference's paracelrun_cpp_proxy), starts ``-w`` worker processes with
``--server_info <endpoints> --cfg_file <cfg>`` (and RANK / WORLD_SIZE / MASTER_* for the process
group), logs the three command lines to ``./paracelrun_log``, watches the workers, and stops the
servers when the workers are done.  If a worker dies the rest of the job is terminated cleanly
(SIGTERM, then SIGKILL after a grace period) instead of being left to hang.

``-m local`` runs everything on this host.  ``-m cluster`` places processes on the hosts of
``--hostfile`` / ``--hostfile_server`` through ``paracel_b200.launch.cluster`` (the reference's
``mpi`` and ``mesos`` modes need MPI and Mesos; their scheduling logic -- gang launch, retry,
watchdogs -- is in that module).  An algorithm name known to ``paracel_b200.run`` may be given
instead of an executable."""
from __future__ import annotations

import argparse
import logging
import os
import signal
import subprocess
import sys
import threading
import time
from typing import List, Optional

from .._core import core
from ..utils.types import SEPERATOR
from .local import free_port

logger = logging.getLogger("paracelrun")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="prun", description="paracel_b200 job launcher")
    ap.add_argument("-p", "--snum", type=int, default=1, help="number of parameter servers")
    ap.add_argument("-w", "--wnum", type=int, default=1, help="number of workers")
    ap.add_argument("-m", "--method", default="local", choices=["local", "cluster", "mpi", "mesos"])
    ap.add_argument("--m_server", default=None, help="launch method of the servers (default: as -m)")
    ap.add_argument("--ppn", type=int, default=1, help="worker processes per node")
    ap.add_argument("--ppn_server", type=int, default=1)
    ap.add_argument("--mem_limit", type=int, default=0, help="MB per worker (0: unlimited)")
    ap.add_argument("--mem_limit_server", type=int, default=0)
    ap.add_argument("--hostfile", default=None)
    ap.add_argument("--hostfile_server", default=None)
    ap.add_argument("-g", "--group", default=None)
    ap.add_argument("--group_server", default=None)
    ap.add_argument("-c", "--cfg_file", default="")
    ap.add_argument("--init_port", type=int, default=0, help="rendezvous port (0: pick a free one)")
    ap.add_argument("--timeout", type=float, default=24 * 3600.0, help="job timeout in seconds")
    ap.add_argument("--gpu", action="store_true", help="one GPU per worker (LOCAL_RANK = CUDA device)")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="algorithm name or executable + args")
    return ap


def _log_cmd(cmd: List[str]) -> None:
    """Append the command line to the run log (the reference's prun.py writes ``paracelrun_log``
    in the working directory).  ``PARACEL_RUN_LOG`` names another file; an empty value
    switches the log off."""
    path = os.environ.get("PARACEL_RUN_LOG", "paracelrun_log")
    if not path:
        return
    with open(path, "a") as f:
        f.write(" ".join(cmd) + "\n")


def start_servers(n: int, host: str = "127.0.0.1", init_port: int = 0, timeout_s: float = 60.0):
    """Start n server daemons and return (processes, 'host:port_PARACEL_host:port')."""
    procs: List[subprocess.Popen] = []
    port_box = {}
    got: List[str] = []
    err: List[BaseException] = []
    listening = threading.Event()

    def on_listening(p):
        port_box["p"] = p
        listening.set()

    def collect():
        try:
            got.extend(core().collect_endpoints(host, init_port, n, timeout_s, on_listening))
        except BaseException as e:  # noqa: BLE001
            err.append(e)
            listening.set()
    th = threading.Thread(target=collect, daemon=True)
    th.start()
    listening.wait(timeout_s)
    if err:
        raise err[0]
    for _ in range(n):
        cmd = [sys.executable, "-m", "paracel_b200.ps.server", "--start_host", host, "--init_port",
               str(port_box["p"]), "--host", host]
        _log_cmd(cmd)
        procs.append(subprocess.Popen(cmd, stdout=subprocess.DEVNULL, start_new_session=True))
    th.join(timeout_s + 5)
    if err or len(got) != n:
        stop_processes(procs)
        raise RuntimeError(f"only {len(got)} of {n} servers came up: {err[0] if err else ''}")
    return procs, SEPERATOR.join(got)


def stop_processes(procs: List[subprocess.Popen], grace_s: float = 5.0) -> None:
    for p in procs:
        if p.poll() is None:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except (ProcessLookupError, PermissionError):
                p.terminate()
    deadline = time.time() + grace_s
    for p in procs:
        try:
            p.wait(timeout=max(0.1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            try:
                os.killpg(p.pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                p.kill()


def shutdown_servers(server_info: str, procs: List[subprocess.Popen]) -> None:
    from ..ps.client import kvclt
    for ep in server_info.split(SEPERATOR):
        if not ep:
            continue
        h, p = ep.split(":")
        try:
            c = kvclt(h, int(p.split(",")[0]), timeout_s=3.0)
            c.shutdown()
            c.close()
        except Exception:  # noqa: BLE001
            pass
    stop_processes(procs)


def worker_command(command: List[str], server_info: str, cfg_file: str) -> List[str]:
    from ..run import ALGORITHMS
    if command and command[0] in ALGORITHMS:
        base = [sys.executable, "-m", "paracel_b200.run", command[0]] + command[1:]
    elif command and command[0].endswith(".py"):
        base = [sys.executable] + command
    else:
        base = list(command)
    return base + ["--server_info", server_info, "--cfg_file", cfg_file]


def run_workers(cmd: List[str], n: int, timeout_s: float, gpu: bool = False) -> int:
    """Start n ranks of ``cmd`` and watch them; returns the job's exit code."""
    port = free_port()
    procs: List[subprocess.Popen] = []
    for r in range(n):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(n), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        env.setdefault("OMP_NUM_THREADS", "1")
        if gpu:
            env["PCL_USE_GPU"] = "1"
        procs.append(subprocess.Popen(cmd, env=env, start_new_session=True))
    _log_cmd(cmd)
    deadline = time.time() + timeout_s
    rc = 0
    try:
        while True:
            codes = [p.poll() for p in procs]
            bad = [c for c in codes if c not in (None, 0)]
            if bad:
                logger.error("a worker exited with code %s: stopping the job", bad[0])
                rc = int(bad[0]) if bad[0] > 0 else 1
                break
            if all(c == 0 for c in codes):
                break
            if time.time() > deadline:
                logger.error("job timeout after %.0f s", timeout_s)
                rc = 124
                break
            time.sleep(0.2)
    finally:
        stop_processes(procs)
    return rc


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    command = [c for c in a.command if c != "--"]
    if not command:
        print("prun: no command given", file=sys.stderr)
        return 2
    logging.basicConfig(level=logging.INFO, format="%(asctime)s prun %(levelname)s %(message)s")
    if a.method in ("mpi", "mesos"):
        logger.warning("method %s is served by the built-in cluster scheduler", a.method)
        a.method = "cluster"
    if a.method == "cluster":
        from .cluster import run_cluster_job
        return run_cluster_job(a, command)
    servers, info = start_servers(a.snum, init_port=a.init_port)
    try:
        cmd = worker_command(command, info, a.cfg_file)
        return run_workers(cmd, a.wnum, a.timeout, a.gpu)
    finally:
        shutdown_servers(info, servers)


if __name__ == "__main__":
    sys.exit(main())
