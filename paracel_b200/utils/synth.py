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
