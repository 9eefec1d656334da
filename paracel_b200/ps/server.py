"""Starting and stopping host parameter servers (reference:
src/start_server.cpp:20-31 and ``init_thrds``, include/server.hpp:405-459)."""
from __future__ import annotations

import argparse
import socket
import sys
from typing import List, Optional, Tuple

from .._core import core
from .handlers import python_filter_callback, python_update_callback


def make_server():
    srv = core().PsServer()
    srv.set_python_update(python_update_callback)
    srv.set_python_filter(python_filter_callback)
    return srv


class LocalServers:
    """``n`` servers running as threads of this process (tests, serial use)."""

    def __init__(self, n: int = 1, host: str = "127.0.0.1"):
        self.servers = [make_server() for _ in range(n)]
        self.endpoints: List[Tuple[str, int]] = []
        for s in self.servers:
            port = s.start(host, 0)
            self.endpoints.append((host, port))

    def info(self) -> str:
        from ..utils.types import SEPERATOR
        return SEPERATOR.join(f"{h}:{p}" for h, p in self.endpoints)

    def stop(self):
        for s in self.servers:
            s.stop()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.stop()


def report_endpoint(start_host: str, init_port: int, host: str, port: int) -> None:
    """Tell the launcher's rendezvous socket where this server listens and wait for 'done'
    (the role of the REQ/REP exchange in server.hpp:408-442)."""
    with socket.create_connection((start_host, init_port), timeout=60) as s:
        s.sendall(f"{host}:{port}\n".encode())
        s.settimeout(60)
        s.recv(16)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="paracel_b200 parameter server")
    ap.add_argument("--start_host", default="127.0.0.1")
    ap.add_argument("--init_port", type=int, default=0, help="launcher rendezvous port (0: none)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=0)
    args = ap.parse_args(argv)
    srv = make_server()
    port = srv.start(args.host if args.host != "*" else "0.0.0.0", args.port)
    print(f"server listening on {args.host}:{port}", flush=True)
    if args.init_port:
        report_endpoint(args.start_host, args.init_port, args.host, port)
    srv.wait()
    srv.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
