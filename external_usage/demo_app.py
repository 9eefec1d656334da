#!/usr/bin/env python
"""Demo application built against an installed paracel_b200: histogram of word lengths.

Every worker loads its share of the input lines, counts the lengths of its words locally and
pushes the counts with ``paracel_bupdate`` under keys ``len_<n>``; the server applies the
user handler ``add_counts`` from ``demo_handlers``.  Worker 0 then reads everything whose key
passes the user filter ``length_keys`` and writes ``histogram_0`` (key<TAB>count)."""
import argparse
import os
import sys

from paracel_b200.paralg import paralg
from paracel_b200.parallel.comm import Comm, main_env
from paracel_b200.utils.misc import json_parser


class length_histogram(paralg):
    def __init__(self, hosts, comm, cfg):
        super().__init__(hosts, comm, cfg.parse("output"))
        self.input = cfg.check_parse("input")
        self.handle_file = cfg.check_parse("update_file")
        self.update_func = cfg.parse("update_function")
        self.filter_file = cfg.check_parse("filter_file")
        self.filter_func = cfg.parse("filter_function")

    def solve(self):
        local = {}
        for line in self.paracel_load(self.input):
            for w in line.split():
                local[len(w)] = local.get(len(w), 0) + 1
        self.paracel_register_bupdate(self.handle_file, self.update_func)
        for n, c in local.items():
            self.paracel_bupdate(f"len_{n}", c)
        self.paracel_sync()
        if self.get_worker_id() == 0:
            hist = self.paracel_read_special(self.filter_file, self.filter_func)
            self.paracel_dump_dict({k: int(v) for k, v in hist.items()}, "histogram_")
        self.paracel_sync()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--server_info", required=True)
    ap.add_argument("--cfg_file", required=True)
    a = ap.parse_args()
    env = main_env()
    try:
        app = length_histogram(a.server_info, Comm(), json_parser(a.cfg_file))
        app.solve()
    finally:
        env.close()


if __name__ == "__main__":
    sys.exit(main())
