"""LDA by collapsed Gibbs sampling on GPUs with the word-topic counts in HBM (device path
of alg/topic_model/gLDA.hpp:40-500).

``LdaGibbsGpu`` is a ``paralg`` subclass on the device backend.  The word-topic counts are
int32 rows keyed by the word id (the reference's ``<word_id>`` keys, gLDA.hpp:431-441) sharded
over the ranks' HBM, the topic sums the single row ``topic_sums_0``.  Documents are processed
in minibatches; one minibatch step is

    paracel_read_multi(word keys)        wait for the SSP bound, then a sparse keyed pull of
                                         the batch's rows by peer loads
    one Gibbs sweep over the batch       pcl_lda_gibbs (one warp per document)
    paracel_bupdate_multi(word keys, cur, "", "gLDA_word_update", old=pulled)
                                         integer reductions of (current - pulled) at the owner
    iter_commit                          clock word stored into every peer's HBM

which is the reference's push-deltas / sync / pull cycle (gLDA.hpp:429-443) made sparse per
minibatch and bounded-stale instead of bulk synchronous."""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..paralg import paralg


class LdaGibbsGpu(paralg):
    def __init__(self, vocab: int, k_topics: int = 1024, alpha: Optional[float] = None,
                 beta: float = 0.01, iters: int = 10, nbatch: int = 4, staleness: int = 2,
                 group=None, device=None, seed: int = 0, timeout_s: float = 10.0, comm=None,
                 hosts_dct_str=None, output: str = "", word_names=None):
        if k_topics not in (128, 256, 512, 1024):
            raise ValueError("k_topics must be 128, 256, 512 or 1024")
        super().__init__(hosts_dct_str, comm, output, int(iters) * max(1, int(nbatch)), int(staleness),
                         True, wait_timeout_s=timeout_s, backend="gpu", device=device, group=group)
        self.group = group
        self.world, self.rank = self.get_worker_size(), self.get_worker_id()
        self.V, self.K = int(vocab), int(k_topics)
        self.alpha = 50.0 / self.K if alpha is None else float(alpha)
        self.beta = float(beta)
        self.iters, self.nbatch, self.seed = int(iters), max(1, int(nbatch)), seed
        self.wt_tab = self.paracel_row_table(self.V, self.K, dtype=torch.int32, names=word_names,
                                             handler="gLDA_word_update")
        self.ts_tab = self.paracel_row_table(1, self.K, prefix="topic_sums_", dtype=torch.int32,
                                             handler="gLDA_sum_topic_update")
        self.wt, self.ts = self.wt_tab.table, self.ts_tab.table
        self.ll = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._zero_id = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.step_no = 0

    def load_docs(self, doc_ptr: torch.Tensor, words: torch.Tensor):
        """This rank's documents as CSR: ``doc_ptr`` (int64, n_docs + 1) and global word ids."""
        dev, K = self.device, self.K
        doc_ptr = doc_ptr.to(dev, torch.int64).contiguous()
        words = words.to(dev, torch.int64).contiguous()
        self.n_docs = doc_ptr.numel() - 1
        self.T = int(words.numel())
        self.doc_len = (doc_ptr[1:] - doc_ptr[:-1]).to(torch.int32).contiguous()
        _lib.validate_ids(words, 0, self.V, "LDA corpus (word ids)")
        g = torch.Generator(device=dev)
        g.manual_seed(self.seed * 104729 + 13 + self.rank)
        self.z = torch.randint(0, K, (self.T,), device=dev, generator=g, dtype=torch.int32)
        doc_of = torch.repeat_interleave(torch.arange(self.n_docs, device=dev), self.doc_len.long())
        self.n_dk = torch.zeros(self.n_docs, K, dtype=torch.int32, device=dev)
        self.n_dk.view(-1).index_add_(0, doc_of * K + self.z.long(),
                                      torch.ones(self.T, dtype=torch.int32, device=dev))
        # minibatches: contiguous document ranges with about the same number of tokens
        bounds = [0]
        for b in range(1, self.nbatch):
            target = self.T * b // self.nbatch
            bounds.append(int(torch.searchsorted(doc_ptr, torch.tensor([target], device=dev)).item()))
        bounds.append(self.n_docs)
        self.batches = []
        max_vocab = 1
        for b in range(self.nbatch):
            d0, d1 = bounds[b], max(bounds[b + 1], bounds[b])
            t0, t1 = int(doc_ptr[d0].item()), int(doc_ptr[d1].item())
            vocab, widx = torch.unique(words[t0:t1], return_inverse=True)
            self.batches.append({
                "d0": d0, "d1": d1, "t0": t0, "t1": t1,
                "ptr": (doc_ptr[d0:d1 + 1] - t0).contiguous(),
                "vocab": vocab.contiguous(), "widx": widx.to(torch.int32).contiguous(),
                "keys": self.paracel_keys(self.wt_tab, vocab.contiguous())})
            max_vocab = max(max_vocab, vocab.numel())
        self.cur = torch.zeros(max_vocab, K, dtype=torch.int32, device=dev)
        self.old = torch.zeros(max_vocab, K, dtype=torch.int32, device=dev)
        self.nk_cur = torch.zeros(1, K, dtype=torch.int32, device=dev)
        self.nk_old = torch.zeros(1, K, dtype=torch.int32, device=dev)
        # first push: this rank's initial counts
        for bt in self.batches:
            nv = bt["vocab"].numel()
            if nv == 0:
                continue
            cnt = torch.zeros(nv, K, dtype=torch.int32, device=dev)
            zz = self.z[bt["t0"]:bt["t1"]].long()
            cnt.view(-1).index_add_(0, bt["widx"].long() * K + zz,
                                    torch.ones(zz.numel(), dtype=torch.int32, device=dev))
            self.paracel_bupdate_multi(bt["keys"], cnt, "", "gLDA_word_update")
        nk = torch.bincount(self.z.long(), minlength=K).to(torch.int32).view(1, K).contiguous()
        self.k_ts = self.paracel_keys(self.ts_tab, self._zero_id)
        self.paracel_bupdate_multi(self.k_ts, nk, "", "gLDA_sum_topic_update")
        tot = torch.tensor([self.T], dtype=torch.int64, device=dev)
        if self.world > 1:
            dist.all_reduce(tot, group=self.group)
        self.T_total = int(tot.item())
        self._barrier()

    def _barrier(self):
        self.paracel_sync()

    def step(self, with_loglik: bool = False):
        bt = self.batches[self.step_no % self.nbatch]
        it = self.step_no
        self.step_no += 1
        nv = bt["vocab"].numel()
        nd = bt["d1"] - bt["d0"]
        s = _lib.stream_ptr()
        if nv > 0 and nd > 0:
            cur, old = self.cur[:nv], self.old[:nv]
            # the staleness wait precedes the first pull of the step
            self.paracel_read_multi(bt["keys"], out=cur, snapshot=old, use_cache=False)
            self.paracel_read_multi(self.k_ts, out=self.nk_cur, snapshot=self.nk_old, use_cache=False)
            _lib.call("pcl_lda_gibbs", bt["ptr"], bt["widx"], self.z[bt["t0"]:bt["t1"]],
                      self.n_dk[bt["d0"]:bt["d1"]], cur, self.nk_cur, nd, self.K, self.alpha, self.beta,
                      self.V * self.beta, (self.seed * 1000003 + it * 7919 + self.rank) & ((1 << 62) - 1),
                      0, s)
            if with_loglik:
                _lib.call("pcl_lda_loglik", bt["ptr"], bt["widx"], self.n_dk[bt["d0"]:bt["d1"]], cur,
                          self.nk_cur, self.doc_len[bt["d0"]:bt["d1"]], nd, self.K, self.alpha, self.beta,
                          self.V * self.beta, self.ll, s)
            self.paracel_bupdate_multi(bt["keys"], cur, "", "gLDA_word_update", old=old)
            self.paracel_bupdate_multi(self.k_ts, self.nk_cur, "", "gLDA_sum_topic_update", old=self.nk_old)
        elif self._dev_wait_needed(self.clock - self.limit_s):
            self.dev_clock.wait()
        self.iter_commit()

    def iteration(self, with_loglik: bool = False) -> Optional[float]:
        """One pass over all local documents; optionally the global log-likelihood."""
        if with_loglik:
            self.ll.zero_()
        with self.phase("iteration"):
            for _ in range(self.nbatch):
                self.step(with_loglik)
        res = None
        if with_loglik:
            t = self.ll.clone()
            if self.world > 1:
                dist.all_reduce(t, group=self.group)
            res = float(t.item())
        self.log_metrics(iteration=self.step_no // self.nbatch, tokens=self.T, loglik=res,
                         staleness=self.limit_s, minibatches=self.nbatch)
        return res

    def checkpoint_extra(self):
        return {"z": self.z, "n_dk": self.n_dk, "step_no": self.step_no}

    def restore_extra(self, extra):
        self.z.copy_(extra["z"].to(self.device))
        self.n_dk.copy_(extra["n_dk"].to(self.device))
        self.step_no = int(extra["step_no"])

    def fit(self, with_loglik: bool = False) -> List[float]:
        """Run the iterations that are left (all, or the rest after ``load_checkpoint``)."""
        out = []
        for _ in range(self.step_no // self.nbatch, self.iters):
            r = self.iteration(with_loglik)
            if r is not None:
                out.append(r)
        self._barrier()
        self.paracel_check()
        return out

    def perplexity(self, loglik: float) -> float:
        return math.exp(-loglik / max(self.T_total, 1))

    def topic_word_counts(self) -> torch.Tensor:
        """This rank's shard of the word-topic table (rows = owned word ids in owned_ids order)."""
        return self.wt.shard

    def free(self):
        self.wt = self.ts = None
        self.close()
