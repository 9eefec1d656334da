"""Vertex-centric (Pregel-style) layer on the device backend (device counterpart of
``paracel_b200.pregel`` / the reference's include/pregel/vertex.hpp:29-145).

The reference's ``vertex`` class keeps a value and an active flag per local vertex, calls
``compute(neighbor, weight, value)`` for every out-edge of an active vertex (the message travels
to the neighbour's key with a combining update handler), synchronises, reads the combined
messages back (``vote_to_halt``), and stops when no vertex changed anywhere.

Here the program is written on whole edge tensors instead of one edge at a time:

* the value of vertex v is the scalar key ``<v>`` of a table sharded over the ranks' HBM;
* a superstep evaluates ``compute(values of the sources, edge weights)`` for the out-edges of
  the active local vertices in one tensor expression and sends the results with one
  ``paracel_bupdate_multi`` whose handler combines the messages at the owner: ``max`` (atomic
  max at the owner), ``min`` (the table then holds negated values) or ``add``;
* after ``paracel_sync`` the owned values are read back (``paracel_read_multi``), vertices whose
  value changed stay active, and a one-word all-reduce decides whether anybody is still active.

``MaxValueVertices`` is the reference's example program (max_vertex_value_pregel.cpp:28-53),
``ShortestPaths`` a single-source shortest-path program (min-plus) as a second instance.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .paralg import paralg

_NEG = -3.0e38


class vertex_gpu(paralg):
    combine = "max"            # max | min | add

    def __init__(self, n_vertices: int, group=None, device=None, comm=None, hosts_dct_str=None,
                 output: str = "", names=None):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.world, self.rank, self.group = self.get_worker_size(), self.get_worker_id(), group
        self.n, self.names = int(n_vertices), names
        if self.combine not in ("max", "min", "add"):
            raise ValueError("combine must be max, min or add")
        handler = "add" if self.combine == "add" else "max_updater"
        self.tab = self.paracel_scalar_table(self.n, names=names, handler=handler)
        self._sign = -1.0 if self.combine == "min" else 1.0
        self.supersteps = 0

    # ---- the vertex program (override)
    def compute(self, src_value: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """Message sent along every out-edge of an active vertex (tensors over those edges)."""
        return src_value

    def initial_value(self, vertex_rows: torch.Tensor) -> torch.Tensor:
        """Starting value of the local vertices (default: the vertex name, else the row number)."""
        if self.names is not None:
            return torch.as_tensor(self.names, device=self.device)[vertex_rows].to(torch.float32)
        return vertex_rows.to(torch.float32)

    # ---- runtime
    def load_edges(self, src: torch.Tensor, dst: torch.Tensor, weight: Optional[torch.Tensor] = None,
                   init_values: Optional[torch.Tensor] = None):
        """Out-edges (table rows) of the vertices this rank holds."""
        dev = self.device
        self.src, self.dst = src.to(dev, torch.int64), dst.to(dev, torch.int64).contiguous()
        self.wgt = (torch.ones(self.src.numel(), device=dev) if weight is None
                    else weight.to(dev, torch.float32))
        self.lv, self.src_l = torch.unique(self.src, return_inverse=True)
        val = self.initial_value(self.lv) if init_values is None else init_values
        self.val = val.to(dev, torch.float32).contiguous()
        self.k_own = self.paracel_keys(self.tab, self.lv)
        fill = 0.0 if self.combine == "add" else _NEG
        self.paracel_local_shard(self.tab).fill_(fill)
        self.paracel_sync()
        self.paracel_bupdate_multi(self.k_own, (self._sign * self.val).contiguous(), "", None)
        self.paracel_sync()

    def run_supersteps(self, max_steps: int = 1 << 20) -> int:
        active = torch.ones(self.lv.numel(), dtype=torch.bool, device=self.device)
        steps = 0
        while steps < max_steps:
            steps += 1
            sel = active[self.src_l]
            if bool(sel.any()):
                msg = self.compute(self.val[self.src_l[sel]], self.wgt[sel])
                kb = self.paracel_keys(self.tab, self.dst[sel].contiguous())
                self.paracel_bupdate_multi(kb, (self._sign * msg).contiguous(), "", None)
            self.paracel_sync()
            new = self._sign * self.paracel_read_multi(self.k_own, use_cache=False)
            active = new != self.val
            self.val = new
            changed = active.any().to(torch.int32).reshape(1)
            if self.world > 1:
                dist.all_reduce(changed, group=self.group)
            self.paracel_sync()
            if int(changed.item()) == 0:
                break
        self.supersteps = steps
        self.paracel_check()
        return steps

    def values_of(self, vertex_rows: torch.Tensor) -> torch.Tensor:
        """Current values of any vertices (table rows), read from their owners."""
        rows = vertex_rows.to(self.device, torch.int64).contiguous()
        return self._sign * self.paracel_read_multi(self.paracel_keys(self.tab, rows), use_cache=False)

    def dump_result(self, outdir: str = "", prefix: str = "vertex_val_"):
        """``<prefix><rank>``: ``vertex\\tvalue`` for the vertices this rank holds."""
        from .utils.dump import dump_dict_scalar
        outdir = outdir or self.output
        os.makedirs(outdir, exist_ok=True)
        ids = self.lv.cpu().tolist()
        if self.names is not None:
            ids = [self.names[j] for j in ids]
        dump_dict_scalar(dict(zip((str(x) for x in ids), self.val.cpu().tolist())),
                         os.path.join(outdir, f"{prefix}{self.rank}"))
        self.paracel_sync()

    def free(self):
        self.close()


class MaxValueVertices(vertex_gpu):
    """Every vertex ends with the largest value that reaches it along edges."""
    combine = "max"


class ShortestPaths(vertex_gpu):
    """Single-source shortest paths: messages are ``distance(source) + weight``, combined by
    ``min``; vertices start at +3e38 except the source vertex, which starts at 0."""
    combine = "min"

    def __init__(self, n_vertices: int, source_row: int, **kw):
        super().__init__(n_vertices, **kw)
        self.source_row = int(source_row)

    def initial_value(self, vertex_rows):
        v = torch.full((vertex_rows.numel(),), -_NEG, device=self.device)
        v[vertex_rows == self.source_row] = 0.0
        return v

    def compute(self, src_value, weight):
        return src_value + weight
