"""Steady-state inversion.  The reference's parallel class is an empty stub
(alg/misc/steady_state_inversion/steady_state_inversion.hpp:51-57); the working
implementation is the serial tool, see ``paracel_b200.tool.steady_state_inversion_serial``."""
from __future__ import annotations

from ..paralg import paralg


class steady_state_inversion(paralg):
    def __init__(self, comm, hosts_dct_str, input: str = "", output: str = "", **kw):
        super().__init__(hosts_dct_str, comm, output, **kw)
        self.input = input

    def solve(self):
        from ..tool.steady_state_inversion_serial import solve_files
        if self.get_worker_id() == 0 and self.input:
            solve_files(self.input, None, self.output)
        self.paracel_sync()
