"""Synthetic data files for the algorithms (reference: tool/datagen.py:40-202, which uses
scikit-learn generators and downloads sample corpora; there is no network here, so
everything is generated).

    python -m paracel_b200.tool.datagen -m classification -o data.csv -n 10000 -k 100
"""
from __future__ import annotations

import argparse

import numpy as np


def classification(out: str, n: int = 10000, k: int = 100, sep: str = ",", seed: int = 0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, k))
    w = rng.standard_normal(k)
    y = (rng.random(n) < 1 / (1 + np.exp(-X @ w))).astype(float)
    np.savetxt(out, np.concatenate([X, y[:, None]], 1), delimiter=sep, fmt="%.6f")
    return X, y, w


def regression(out: str, n: int = 10000, k: int = 100, sep: str = ",", noise: float = 0.1, seed: int = 0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((n, k))
    w = rng.standard_normal(k)
    y = X @ w + noise * rng.standard_normal(n)
    np.savetxt(out, np.concatenate([X, y[:, None]], 1), delimiter=sep, fmt="%.6f")
    return X, y, w


def kmeans(out: str, n: int = 10000, k: int = 100, ncenters: int = 10, seed: int = 0):
    rng = np.random.default_rng(seed)
    C = rng.uniform(-10, 10, (ncenters, k))
    lab = rng.integers(0, ncenters, n)
    X = C[lab] + rng.standard_normal((n, k))
    with open(out, "w") as f:
        for i in range(n):
            f.write(f"{i}\t" + ",".join("%.6f" % v for v in X[i]) + "\n")
    return X, lab


def lda(out: str, ndocs: int = 1000, vocab: int = 500, topics: int = 10, doc_len: int = 100, seed: int = 0):
    rng = np.random.default_rng(seed)
    phi = rng.dirichlet(np.full(vocab, 0.05), topics)
    with open(out, "w") as f:
        for _ in range(ndocs):
            theta = rng.dirichlet(np.full(topics, 0.3))
            z = rng.choice(topics, doc_len, p=theta)
            f.write(" ".join("w%d" % rng.choice(vocab, p=phi[t]) for t in z) + "\n")


def ratings(out: str, nu: int = 1000, ni: int = 500, nnz: int = 50000, seed: int = 0, mf_format: bool = True):
    rng = np.random.default_rng(seed)
    P, Q = rng.normal(0, 0.5, (nu, 8)), rng.normal(0, 0.5, (ni, 8))
    u, i = rng.integers(0, nu, nnz), rng.integers(0, ni, nnz)
    r = np.clip(np.round(3 + (P[u] * Q[i]).sum(1) + rng.normal(0, 0.5, nnz)), 1, 5)
    with open(out, "w") as f:
        for a, b, c in zip(u, i, r):
            f.write(f"{a} {b} 20140101 {c:.0f}\n" if mf_format else f"{a},{b},{c:.0f}\n")


def graph(out: str, n: int = 1000, m: int = 10000, seed: int = 0):
    rng = np.random.default_rng(seed)
    src = rng.integers(0, n, m)
    dst = (rng.random(m) ** 2 * n).astype(np.int64)
    with open(out, "w") as f:
        for a, b in sorted(set(zip(src.tolist(), dst.tolist()))):
            if a != b:
                f.write(f"{a},{b}\n")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--method", required=True,
                    choices=["classification", "regression", "kmeans", "lda", "ratings", "graph"])
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("-n", "--nsamples", type=int, default=10000)
    ap.add_argument("-k", "--nfeatures", type=int, default=100)
    ap.add_argument("-s", "--sep", default=",")
    a = ap.parse_args(argv)
    if a.method == "classification":
        classification(a.output, a.nsamples, a.nfeatures, a.sep)
    elif a.method == "regression":
        regression(a.output, a.nsamples, a.nfeatures, a.sep)
    elif a.method == "kmeans":
        kmeans(a.output, a.nsamples, a.nfeatures)
    elif a.method == "lda":
        lda(a.output, a.nsamples)
    elif a.method == "ratings":
        ratings(a.output, nnz=a.nsamples)
    else:
        graph(a.output, a.nfeatures, a.nsamples)


if __name__ == "__main__":
    main()
