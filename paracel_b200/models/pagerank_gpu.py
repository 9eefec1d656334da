"""PageRank with the rank vector sharded in HBM (device path of
alg/graph_alg/pagerank/pr.hpp:40-200).

Vertices are dense ids in [0, n); rank r owns the range ``[r*S, (r+1)*S)`` and keeps the
in-links of its vertices as CSR.  What travels between ranks is the contribution vector
``c(u) = pr(u) / outdeg(u)``.  ``PageRankGpu`` is a ``paralg`` subclass on the device backend
with two dense keys, ``pr_contrib_0`` and ``pr_contrib_1``; an iteration is
``paracel_read`` of the current key (all-gather of all shards by peer loads) and one pull
kernel that evaluates ``pr(v) = (1 - d) + d * sum_{u->v} c(u)`` and writes the new
contribution of every owned vertex straight into this rank's shard of the OTHER key
(``paracel_local_shard`` + ``paracel_commit_write``: the reference's read_multi +
write_multi, pr.hpp:140-168).  Out-degrees are reduced with a collective ``paracel_bupdate``
(add handler).  An edge whose target is the sentinel 2147483648 only marks its source as a
vertex with out-links."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.linear import pagerank_pull, pagerank_pull_stream, pagerank_stream_plan
from ..paralg import paralg
from ..utils.types import SENTINEL


class PageRankGpu(paralg):
    KEYS = ("pr_contrib_0", "pr_contrib_1")

    def __init__(self, n_vertices: int, damping: float = 0.85, group=None, device=None,
                 threads_per_row: int = 8, edge_balanced: bool = True, comm=None,
                 hosts_dct_str=None, output: str = ""):
        super().__init__(hosts_dct_str, comm, output, backend="gpu", device=device, group=group)
        self.group = group
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.n, self.d = int(n_vertices), float(damping)
        self.tables = [self.paracel_dense_table(k, self.n, handler="add").table for k in self.KEYS]
        self.S = self.tables[0].S
        self.lo, self.hi = self.tables[0].owned_range()
        self.n_local = max(0, self.hi - self.lo)
        self.tpr = threads_per_row
        self.edge_balanced = edge_balanced
        self.it = 0
        self.delta_l1 = torch.zeros(1, dtype=torch.float64, device=self.device)

    def owner_of(self, v: torch.Tensor) -> torch.Tensor:
        return torch.clamp(v // self.S, max=self.world - 1)

    def load_edges(self, src: torch.Tensor, dst: torch.Tensor):
        """Edges whose destination this rank owns (plus sentinel edges of any source); the
        out-degree of every vertex is summed over all ranks through the parameter table."""
        dev = self.device
        src = src.to(dev, torch.int64)
        dst = dst.to(dev, torch.int64)
        k0 = self.KEYS[0]
        _lib.validate_ids(src, 0, self.n, "PageRank edges (source ids)")
        _lib.validate_ids(dst, 0, self.n, "PageRank edges (target ids)", skip=SENTINEL)
        # out-degrees: reduce-scatter(add) of the local source counts
        self.paracel_write(k0, torch.zeros(self.n, device=dev))
        self.paracel_delta_buffer(k0).copy_(torch.bincount(src, minlength=self.n).to(torch.float32))
        self.paracel_bupdate(k0, self.paracel_delta_buffer(k0), "", "add", collective=True)
        outdeg_full = self.paracel_read(k0).clone()
        self._barrier()
        real = dst != SENTINEL
        src, dst = src[real], dst[real]
        assert bool(((dst >= self.lo) & (dst < self.hi)).all()), "edges must be placed by destination owner"
        order = torch.argsort(dst, stable=True)
        self.cols = src[order].to(torch.int32).contiguous()
        counts = torch.bincount(dst - self.lo, minlength=self.n_local)
        self.row_ptr = torch.zeros(self.n_local + 1, dtype=torch.int64, device=dev)
        self.row_ptr[1:] = torch.cumsum(counts, 0)
        self.n_edges_local = int(self.cols.numel())
        self.heavy_deg = 2048
        self.heavy_rows = torch.nonzero(counts > self.heavy_deg).flatten().to(torch.int32).contiguous()
        od = outdeg_full[self.lo:self.hi]
        self.inv_outdeg = torch.where(od > 0, 1.0 / od.clamp(min=1.0), torch.zeros_like(od)).contiguous()
        self.has_out = od > 0
        N = int((outdeg_full[: self.n] > 0).sum().item())
        self.N = N
        init = 1.0 / max(N, 1)
        self.rank_local = torch.where(self.has_out, torch.full_like(od, init), torch.zeros_like(od))
        self.rank_new = torch.empty_like(self.rank_local)
        self.acc = torch.zeros(max(self.n_local, 1), device=dev)
        self.plan = self._choose_plan()
        # contribution table for iteration 0 lives in tables[0]
        for k in self.KEYS:
            self.paracel_local_shard(k).zero_()
        self.paracel_local_shard(k0)[: self.n_local] = self.rank_local * self.inv_outdeg
        self.paracel_commit_write(k0)
        self.it = 0

    def _choose_plan(self):
        """Edge-balanced kernel with 2048 or 4096 in-links per block: whichever is faster on this
        graph (the labelling decides; one timed launch each on scratch outputs).  All ranks take
        the choice of the slowest rank's best, so the iteration stays balanced."""
        forced = int(os.environ.get("PCL_PAGERANK_CAP", "0"))
        plans = {cap: pagerank_stream_plan(self.row_ptr, cap) for cap in ((forced,) if forced else (2048, 4096))}
        if len(plans) == 1 or self.n_edges_local == 0 or not self.edge_balanced:
            return next(iter(plans.values()))
        dev = self.device
        probe = torch.full((self.tables[0].L,), 1.0 / max(self.n, 1), device=dev)
        out_c, out_r = torch.empty_like(self.rank_local), torch.empty_like(self.rank_local)
        times = torch.zeros(2, dtype=torch.float64, device=dev)
        for j, cap in enumerate((2048, 4096)):
            for rep in range(2):                       # the second launch is the timed one
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                pagerank_pull_stream(self.row_ptr, self.cols, probe, self.inv_outdeg, self.d, self.acc,
                                     out_c, out_r, None, None, plans[cap])
                e1.record()
                torch.cuda.synchronize(dev)
                times[j] = e0.elapsed_time(e1)
        if self.world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX, group=self.group)
        return plans[2048] if float(times[0]) <= float(times[1]) else plans[4096]

    def _barrier(self):
        self.paracel_sync()

    def step(self, track_delta: bool = False):
        kcur, knxt = self.KEYS[self.it % 2], self.KEYS[(self.it + 1) % 2]
        cur, nxt = self.tables[self.it % 2], self.tables[(self.it + 1) % 2]
        # the pull kernel writes the OTHER key, so a single rank may read its shard in place
        contrib = cur.read(copy=False) if self.world == 1 else self.paracel_read(kcur)
        if track_delta:
            self.delta_l1.zero_()
        if self.edge_balanced:
            pagerank_pull_stream(self.row_ptr, self.cols, contrib, self.inv_outdeg, self.d, self.acc,
                                 nxt.shard, self.rank_new, self.delta_l1 if track_delta else None,
                                 self.rank_local if track_delta else None, self.plan)
        else:
            pagerank_pull(self.row_ptr, self.cols, contrib, self.inv_outdeg, self.d,
                          nxt.shard, self.rank_new, self.delta_l1 if track_delta else None,
                          self.rank_local if track_delta else None, self.tpr,
                          self.heavy_rows if self.heavy_rows.numel() else None, self.heavy_deg)
        self.paracel_commit_write(knxt)
        self.rank_local, self.rank_new = self.rank_new, self.rank_local
        self.it += 1

    def checkpoint_extra(self):
        return {"rank_local": self.rank_local, "it": self.it}

    def restore_extra(self, extra):
        self.rank_local.copy_(extra["rank_local"].to(self.device))
        self.it = int(extra["it"])

    def run(self, rounds: int):
        for _ in range(rounds):
            with self.phase("iteration"):
                self.step()
            self.log_metrics(iteration=self.it, edges=self.n_edges_local)
        self._barrier()
        self.paracel_check()

    def ranks(self) -> torch.Tensor:
        """Ranks of the owned vertices (vertices without out-links are reported as well)."""
        return self.rank_local[: self.n_local]

    def dump_result(self, outdir: str, names=None):
        """``pagerank_0``: ``vertex\\trank`` for every vertex that has out-links (pr.hpp:184-193);
        ``names`` (array indexed by the dense vertex id) gives the ids to print."""
        from ..utils.dump import dump_dict_scalar
        os.makedirs(outdir, exist_ok=True)
        self._barrier()
        ids = (torch.nonzero(self.has_out).flatten() + self.lo).cpu().tolist()
        if names is not None:
            ids = [int(names[j]) for j in ids]
        vals = self.rank_local[self.has_out].cpu().tolist()
        part = dict(zip(ids, vals))
        parts = [part]
        if self.world > 1:
            parts = [None] * self.world
            dist.all_gather_object(parts, part, group=self.group)
        if self.rank == 0:
            with open(os.path.join(outdir, "pagerank_0"), "w") as f:
                for p in parts:
                    dump_dict_scalar(p, f)
        self._barrier()

    def free(self):
        self.tables = []
        self.close()
