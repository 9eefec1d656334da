"""Seeded synthetic data generators for the benchmark configurations (the
reference only ships sklearn toy generators and sample downloads,
tool/datagen.py:40-202).  Everything is generated in fixed-size chunks whose
random streams depend only on (seed, chunk index), so any number of ranks can
regenerate the identical global dataset and keep its own part."""
from __future__ import annotations

from typing import Iterator, Tuple

import torch


def zipf_cdf(n: int, s: float, device) -> torch.Tensor:
    """CDF of the bounded Zipf law p(k) ~ k^-s, k = 1..n (float64)."""
    k = torch.arange(1, n + 1, dtype=torch.float64, device=device)
    w = k.pow(-s)
    c = torch.cumsum(w, 0)
    return c / c[-1]


def zipf_draw(cdf: torch.Tensor, m: int, gen: torch.Generator) -> torch.Tensor:
    """m ids in [0, n) with id = Zipf rank - 1."""
    x = torch.rand(m, dtype=torch.float64, device=cdf.device, generator=gen)
    return torch.searchsorted(cdf, x).clamp_(max=cdf.numel() - 1)


class MfRatingStream:
    """Ratings r = round(clip(p_u . q_i + N(0, noise), 1, 5)) for (u, i) drawn
    independently from Zipf(s) laws, with rank-``latent`` N(0, 0.5) factors."""

    def __init__(self, n_users: int, n_items: int, nnz: int, s: float = 1.1, latent: int = 16,
                 noise: float = 0.5, seed: int = 0, device="cuda", chunk: int = 1 << 24):
        self.n_users, self.n_items, self.nnz = n_users, n_items, nnz
        self.device = torch.device(device)
        self.chunk = chunk
        self.seed = seed
        self.noise = noise
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        self.P = 0.5 * torch.randn(n_users, latent, device=self.device, generator=g)
        self.Q = 0.5 * torch.randn(n_items, latent, device=self.device, generator=g)
        self.cdf_u = zipf_cdf(n_users, s, self.device)
        self.cdf_i = zipf_cdf(n_items, s, self.device)

    def nchunks(self) -> int:
        return (self.nnz + self.chunk - 1) // self.chunk

    def chunk_at(self, c: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        m = min(self.chunk, self.nnz - c * self.chunk)
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 1000003 + 7 + c)
        u = zipf_draw(self.cdf_u, m, g)
        i = zipf_draw(self.cdf_i, m, g)
        dot = (self.P[u] * self.Q[i]).sum(1)
        r = dot + self.noise * torch.randn(m, device=self.device, generator=g)
        r = torch.round(r.clamp_(1.0, 5.0))
        return u, i, r

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
        for c in range(self.nchunks()):
            yield self.chunk_at(c)

    def counts(self) -> Tuple[torch.Tensor, torch.Tensor]:
        cu = torch.zeros(self.n_users, dtype=torch.int64, device=self.device)
        ci = torch.zeros(self.n_items, dtype=torch.int64, device=self.device)
        for u, i, _ in self:
            cu += torch.bincount(u, minlength=self.n_users)
            ci += torch.bincount(i, minlength=self.n_items)
        return cu, ci


class SparseLrStream:
    """Rows with ``nnz_row`` features drawn Zipf(s) over ``n_features`` hashed ids (value 1.0);
    labels Bernoulli(sigmoid(w.x)) for a sparse true w (``w_density`` non-zeros, N(0, 1))."""

    def __init__(self, n_rows: int, n_features: int, nnz_row: int = 40, s: float = 1.05,
                 w_density: float = 0.01, seed: int = 0, device="cuda", chunk_rows: int = 1 << 20):
        self.n_rows, self.F, self.k, self.seed = n_rows, n_features, nnz_row, seed
        self.device = torch.device(device)
        self.chunk_rows = chunk_rows
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        self.cdf = zipf_cdf(n_features, s, self.device)
        self.w = torch.zeros(n_features, device=self.device)
        nz = torch.randperm(n_features, device=self.device, generator=g)[: max(1, int(n_features * w_density))]
        self.w[nz] = torch.randn(nz.numel(), device=self.device, generator=g)

    def nchunks(self) -> int:
        return (self.n_rows + self.chunk_rows - 1) // self.chunk_rows

    def chunk_at(self, c: int):
        """(cols int32 [m * k], y fp32 [m]) of chunk c."""
        m = min(self.chunk_rows, self.n_rows - c * self.chunk_rows)
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 1000003 + 11 + c)
        cols = zipf_draw(self.cdf, m * self.k, g).view(m, self.k)
        z = self.w[cols].sum(1)
        y = (torch.rand(m, device=self.device, generator=g) < torch.sigmoid(z)).float()
        return cols.to(torch.int32).reshape(-1), y


def lda_corpus_chunk(n_docs: int, vocab: int, s: float, mean_len: float, seed: int, device):
    """(doc_ptr int64, word ids int64) for ``n_docs`` documents: lengths Poisson(mean_len)
    (at least 1), word ids Zipf(s)."""
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    lens = torch.poisson(torch.full((n_docs,), float(mean_len), device=device), generator=g).long().clamp(min=1)
    ptr = torch.zeros(n_docs + 1, dtype=torch.int64, device=device)
    ptr[1:] = torch.cumsum(lens, 0)
    cdf = zipf_cdf(vocab, s, device)
    words = zipf_draw(cdf, int(ptr[-1].item()), g)
    return ptr, words


def scramble_vertex_blocks(v: torch.Tensor, scale: int, block_log: int = 10) -> torch.Tensor:
    """Bijection on [0, 2^scale) that keeps blocks of 2^block_log consecutive ids together and
    moves block b to (b * odd constant) mod 2^(scale - block_log).  R-MAT skews every id bit the
    same way, so equal id ranges carry very unequal edge counts; after this relabelling the top
    bits depend on all bits of the block number and equal ranges are balanced, while the
    locality inside a block (4 KB of an fp32 vector) is unchanged."""
    if scale <= block_log:
        return v
    hb = scale - block_log
    blk = v >> block_log
    off = v & ((1 << block_log) - 1)
    nb = (blk * 0x9E3779B1) & ((1 << hb) - 1)
    return (nb << block_log) | off


def rmat_edges_chunk(scale: int, m: int, a: float, b: float, c: float, seed: int, device):
    """``m`` edges of an R-MAT graph with 2^scale vertices (quadrant probabilities a, b, c,
    1-a-b-c): (src, dst) int64."""
    device = torch.device(device)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    src = torch.zeros(m, dtype=torch.int64, device=device)
    dst = torch.zeros(m, dtype=torch.int64, device=device)
    for lvl in range(scale):
        r = torch.rand(m, device=device, generator=g)
        right = ((r >= a) & (r < a + b)) | (r >= a + b + c)     # quadrants b and d: dst bit set
        down = r >= a + b                                        # quadrants c and d: src bit set
        src = (src << 1) | down.long()
        dst = (dst << 1) | right.long()
    return src, dst
