"""Rendezvous proxy as a stand-alone program (src/paracelrun_cpp_proxy.cpp:23-35): listens on
``--init_port``, takes one ``host:ports`` line from each of ``--nsrv`` servers, answers each of
them, and prints the lines joined by the endpoint separator for the launcher to read.

    python -m paracel_b200.launch.proxy --nsrv 2 --init_port 7773
"""
from __future__ import annotations

import argparse
import sys

from .._core import core
from ..utils.types import DEFAULT_PORT, SEPERATOR


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="paracel_b200.launch.proxy")
    ap.add_argument("--nsrv", type=int, default=1)
    ap.add_argument("--init_port", type=int, default=DEFAULT_PORT)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args(argv)
    eps = core().collect_endpoints(a.host, a.init_port, a.nsrv, a.timeout, None)
    sys.stdout.write(SEPERATOR.join(eps))
    sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
