"""Max-vertex-value on GPUs (device path of
alg/graph_alg/max_vertex_value/max_vertex_value.hpp:70-121).

``MvvGpu`` is a ``paralg`` subclass on the device backend: the value of vertex v is the scalar
key ``<v>`` of a table sharded over the ranks' HBM with the ``max_updater`` handler.  A round
pushes the value of every active local vertex to its out-neighbours
(``paracel_bupdate_multi`` = system-scope atomic max at the owner), synchronises, reads the
owned values back and keeps the vertices whose value changed active; the run ends when no
vertex changed anywhere."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..paralg import paralg


class MvvGpu(paralg):
    def __init__(self, n_vertices: int, group=None, device=None, comm=None, hosts_dct_str=None,
                 output: str = "", names=None, update_func: str = "max_updater"):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.world, self.rank, self.group = self.get_worker_size(), self.get_worker_id(), group
        self.n, self.names, self.update_func = int(n_vertices), names, update_func
        self.tab = self.paracel_scalar_table(self.n, names=names, handler=update_func)

    def load_edges(self, src: torch.Tensor, dst: torch.Tensor, init_values: Optional[torch.Tensor] = None):
        """Edges (table rows) whose source this rank holds; ``init_values[v]`` (default: the
        vertex name, else the row number) is the starting value of local source v."""
        dev = self.device
        self.src, self.dst = src.to(dev, torch.int64), dst.to(dev, torch.int64)
        self.lv, self.src_l = torch.unique(self.src, return_inverse=True)
        if init_values is None:
            if self.names is not None:
                init_values = torch.as_tensor(self.names, device=dev)[self.lv].to(torch.float32)
            else:
                init_values = self.lv.to(torch.float32)
        self.val = init_values.to(dev, torch.float32).contiguous()
        self.k_own = self.paracel_keys(self.tab, self.lv)
        self.k_dst = self.paracel_keys(self.tab, self.dst.contiguous())
        self.paracel_local_shard(self.tab).fill_(-3.0e38)
        self.paracel_sync()
        self.paracel_bupdate_multi(self.k_own, self.val, "", self.update_func)
        self.paracel_sync()

    def solve(self, max_rounds: int = 1 << 20) -> int:
        dev = self.device
        active = torch.ones(self.lv.numel(), dtype=torch.bool, device=dev)
        rounds = 0
        while rounds < max_rounds:
            rounds += 1
            sel = active[self.src_l]
            if bool(sel.any()):
                kb = self.paracel_keys(self.tab, self.dst[sel].contiguous())
                self.paracel_bupdate_multi(kb, self.val[self.src_l[sel]].contiguous(), "", self.update_func)
            self.paracel_sync()
            new = self.paracel_read_multi(self.k_own, use_cache=False)
            active = new != self.val
            self.val = new
            changed = active.any().to(torch.int32).reshape(1)
            if self.world > 1:
                dist.all_reduce(changed, group=self.group)
            self.paracel_sync()
            if int(changed.item()) == 0:
                break
        self.paracel_check()
        return rounds

    def dump_result(self, outdir: str = ""):
        """``vertex_val_<rank>``: ``vertex\\tvalue`` for the vertices this rank holds."""
        from ..utils.dump import dump_dict_scalar
        outdir = outdir or self.output
        os.makedirs(outdir, exist_ok=True)
        ids = self.lv.cpu().tolist()
        if self.names is not None:
            ids = [self.names[j] for j in ids]
        dump_dict_scalar(dict(zip((str(x) for x in ids), self.val.cpu().tolist())),
                         os.path.join(outdir, f"vertex_val_{self.rank}"))
        self.paracel_sync()

    def free(self):
        self.close()
