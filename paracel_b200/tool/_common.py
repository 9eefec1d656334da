from __future__ import annotations

import sys

from ..parallel.comm import Comm
from ..paralg import paralg


def serial_paralg(output: str) -> paralg:
    """paralg in its direct-usage form (no servers, communicator of size 1)."""
    return paralg(Comm(), output=output)


def cli(main):
    if len(sys.argv) != 3 or sys.argv[1] != "--cfg_file":
        print("usage: python -m <tool> --cfg_file cfg.json", file=sys.stderr)
        return 2
    return main(sys.argv[2]) or 0
