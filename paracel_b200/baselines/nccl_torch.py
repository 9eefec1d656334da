"""NCCL-only PyTorch baselines of the sparse L1-LR, LDA and PageRank configurations: the same
algorithms written with stock PyTorch ops and NCCL collectives (``all_gather_into_tensor``,
``reduce_scatter_tensor``, ``all_reduce``) only.  They exist to be measured against."""
from __future__ import annotations

import torch
import torch.distributed as dist


class _Base:
    def __init__(self, group=None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")

    def _all_gather(self, shard):
        if self.world == 1:
            return shard
        out = torch.empty(shard.numel() * self.world, dtype=shard.dtype, device=self.device)
        dist.all_gather_into_tensor(out, shard.contiguous(), group=self.group)
        return out

    def _reduce_scatter(self, full):
        if self.world == 1:
            return full
        out = torch.empty(full.numel() // self.world, dtype=full.dtype, device=self.device)
        dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
        return out


class SparseLinearNcclTorch(_Base):
    def __init__(self, n_features, eta=0.5, lam=1e-6, nbatch=1, group=None, device=None, **_):
        super().__init__(group, device)
        self.F, self.eta, self.lam, self.nbatch = n_features, eta, lam, nbatch
        self.S = (n_features + self.world - 1) // self.world
        self.theta = torch.zeros(self.S, device=self.device)
        self.loss = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.step_no = 0

    def load(self, row_ptr, cols, y, vals=None):
        self.k = int((row_ptr[1] - row_ptr[0]).item())
        self.cols = cols.long().view(-1, self.k)
        self.y = y
        n = torch.tensor([y.numel()], dtype=torch.int64, device=self.device)
        if self.world > 1:
            dist.all_reduce(n, group=self.group)
        self.n_total = int(n)
        b = torch.linspace(0, y.numel(), self.nbatch + 1).long().tolist()
        self.batches = list(zip(b[:-1], b[1:]))

    def step(self):
        lo, hi = self.batches[self.step_no % self.nbatch]
        self.step_no += 1
        theta = self._all_gather(self.theta)[: self.F]
        C = self.cols[lo:hi]
        z = theta[C].sum(1)
        h = torch.sigmoid(z)
        r = self.y[lo:hi] - h
        self.loss = -(self.y[lo:hi] * torch.log(h.clamp(1e-7, 1 - 1e-7))
                      + (1 - self.y[lo:hi]) * torch.log((1 - h).clamp(1e-7, 1))).double().sum().view(1)
        g = torch.zeros(self.S * self.world, device=self.device)
        g.index_add_(0, C.reshape(-1), r[:, None].expand(-1, self.k).reshape(-1))
        gs = self._reduce_scatter(g)
        nb = self.n_total / self.nbatch
        w = self.theta + (self.eta / nb) * gs
        t = (self.eta / nb) * self.lam
        self.theta = torch.sign(w) * torch.clamp(w.abs() - t, min=0)

    def mean_loss(self):
        t = self.loss.clone()
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return float(t) / max(self.n_total / self.nbatch, 1.0)

    def nnz_weights(self):
        t = (self.theta != 0).sum().double().view(1)
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return int(t)


class PageRankNcclTorch(_Base):
    def __init__(self, n_vertices, damping=0.85, group=None, device=None, **_):
        super().__init__(group, device)
        self.n, self.d = n_vertices, damping
        self.S = ((n_vertices + self.world - 1) // self.world + 3) // 4 * 4
        self.lo = self.rank * self.S
        self.hi = min(self.n, self.lo + self.S)

    def owner_of(self, v):
        return torch.clamp(v // self.S, max=self.world - 1)

    def load_edges(self, src, dst):
        dev = self.device
        od = torch.bincount(src, minlength=self.S * self.world).float()
        if self.world > 1:
            dist.all_reduce(od, group=self.group)
        self.n_edges_local = int(src.numel())
        order = torch.argsort(dst, stable=True)
        self.cols = src[order]
        counts = torch.bincount(dst - self.lo, minlength=self.S)
        crow = torch.zeros(self.S + 1, dtype=torch.int64, device=dev)
        crow[1:] = torch.cumsum(counts, 0)
        self.A = torch.sparse_csr_tensor(crow, self.cols, torch.ones(self.cols.numel(), device=dev),
                                         size=(self.S, self.S * self.world))
        odl = od[self.lo:self.lo + self.S]
        self.inv = torch.where(odl > 0, 1.0 / odl.clamp(min=1), torch.zeros_like(odl))
        N = int((od > 0).sum())
        self.contrib = torch.where(odl > 0, torch.full_like(odl, 1.0 / max(N, 1)), torch.zeros_like(odl)) * self.inv

    def step(self):
        full = self._all_gather(self.contrib)
        s = torch.mv(self.A, full)
        pr = (1.0 - self.d) + self.d * s
        self.rank_local = pr
        self.contrib = pr * self.inv


class LdaNcclTorch(_Base):
    """Minibatch "parallel Gibbs" with torch.multinomial: every token of the minibatch is resampled
    from counts frozen at the start of the minibatch, counts are all-reduced afterwards."""

    def __init__(self, vocab, k_topics, alpha=None, beta=0.01, nbatch=4, group=None, device=None, **_):
        super().__init__(group, device)
        self.V, self.K, self.beta, self.nbatch = vocab, k_topics, beta, nbatch
        self.alpha = 50.0 / k_topics if alpha is None else alpha
        self.step_no = 0

    def load_docs(self, doc_ptr, words):
        dev = self.device
        self.words = words.to(dev)
        lens = doc_ptr[1:] - doc_ptr[:-1]
        self.doc_of = torch.repeat_interleave(torch.arange(lens.numel(), device=dev), lens)
        T = words.numel()
        self.z = torch.randint(0, self.K, (T,), device=dev)
        self.n_dk = torch.zeros(lens.numel(), self.K, dtype=torch.int32, device=dev)
        self.n_dk.view(-1).index_add_(0, self.doc_of * self.K + self.z, torch.ones(T, dtype=torch.int32, device=dev))
        self.n_wk = torch.zeros(self.V, self.K, dtype=torch.int32, device=dev)
        self.n_wk.view(-1).index_add_(0, self.words * self.K + self.z, torch.ones(T, dtype=torch.int32, device=dev))
        if self.world > 1:
            dist.all_reduce(self.n_wk, group=self.group)
        b = [T * i // self.nbatch for i in range(self.nbatch + 1)]
        self.batches = list(zip(b[:-1], b[1:]))

    def step(self, chunk=1 << 18):
        lo, hi = self.batches[self.step_no % self.nbatch]
        self.step_no += 1
        n_k = self.n_wk.sum(0).float()
        delta = torch.zeros_like(self.n_wk)
        for s in range(lo, hi, chunk):
            e = min(hi, s + chunk)
            w, d, zo = self.words[s:e], self.doc_of[s:e], self.z[s:e]
            p = (self.n_dk[d].float() + self.alpha) * (self.n_wk[w].float() + self.beta) / (n_k + self.V * self.beta)
            zn = torch.multinomial(p, 1).squeeze(1)
            one = torch.ones(e - s, dtype=torch.int32, device=self.device)
            self.n_dk.view(-1).index_add_(0, d * self.K + zo, -one)
            self.n_dk.view(-1).index_add_(0, d * self.K + zn, one)
            delta.view(-1).index_add_(0, w * self.K + zo, -one)
            delta.view(-1).index_add_(0, w * self.K + zn, one)
            self.z[s:e] = zn
        if self.world > 1:
            dist.all_reduce(delta, group=self.group)
        self.n_wk += delta
