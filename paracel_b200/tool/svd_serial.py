"""Serial truncated SVD (reference: tool/svd_serial.cpp:40-193): alternating least squares
factorisation, Cholesky-QR of both factors, SVD of the small core, dumps SIGMA_0, U_0, V_0."""
from __future__ import annotations

from ..models.svd import svd as _svd
from ..parallel.comm import Comm
from ..ps.server import LocalServers
from ..utils.misc import json_parser
from ._common import cli


def solve(input: str, output: str, k: int, iters: int = 10, seed: int = 0):
    with LocalServers(1) as ls:
        s = _svd(Comm(), ls.info(), input, output, k=k, iters=iters, seed=seed)
        s.solve()
        s.dump_result()
        s.close()
        return s


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    solve(pt.check_parse("input", str), pt.parse("output", str), pt.parse("k", int))


if __name__ == "__main__":
    raise SystemExit(cli(main))
