"""Serial collapsed-Gibbs LDA with a dense topic-word table (reference:
tool/gLDA_serial.cpp:40-391): the same sampler as the parallel model on one process."""
from __future__ import annotations

import math
import os

import numpy as np

from .._core import core
from ..utils.misc import json_parser
from ._common import cli, serial_paralg


class gLDA_serial:
    def __init__(self, input: str, output: str, alpha: float, beta: float, k_topics: int, iters: int,
                 top_words: int = 10, seed: int = 0):
        self.pt = serial_paralg("")
        self.input, self.output = input, output
        self.alpha, self.beta, self.K, self.iters, self.top = alpha, beta, int(k_topics), int(iters), top_words
        self.seed = seed

    def solve(self):
        docs = [l.split() for l in self.pt.paracel_loadall(self.input)]
        self.word2id = {}
        for d in docs:
            for w in d:
                self.word2id.setdefault(w, len(self.word2id))
        self.id2word = {i: w for w, i in self.word2id.items()}
        V, K = len(self.word2id), self.K
        lens = np.asarray([len(d) for d in docs], dtype=np.int32)
        ptr = np.zeros(len(docs) + 1, dtype=np.int64)
        np.cumsum(lens, out=ptr[1:])
        words = np.fromiter((self.word2id[w] for d in docs for w in d), dtype=np.int32, count=int(ptr[-1]))
        rng = np.random.default_rng(self.seed)
        z = rng.integers(0, K, size=words.size, dtype=np.int32)
        nd = np.zeros((len(docs), K), dtype=np.int32)
        np.add.at(nd, (np.repeat(np.arange(len(docs)), lens), z), 1)
        nw = np.zeros((V, K), dtype=np.int32)
        np.add.at(nw, (words, z), 1)
        nk = np.bincount(z, minlength=K).astype(np.int32)
        self.loglik = []
        for it in range(self.iters):
            core().lda_gibbs_sweep(ptr, words, z, nd, nw, nk, lens, K, V, self.alpha, self.beta,
                                   self.seed * 7919 + it)
            theta = (nd + self.alpha) / (lens[:, None] + K * self.alpha)
            phi = (nw + self.beta) / (nk[None, :] + V * self.beta)
            doc_of = np.repeat(np.arange(len(docs)), lens)
            self.loglik.append(float(np.log((theta[doc_of] * phi[words]).sum(1) + 1e-300).sum()))
        self.nw, self.nk, self.V, self.T = nw, nk, V, int(words.size)

    def perplexity(self) -> float:
        return math.exp(-self.loglik[-1] / max(self.T, 1))

    def save(self):
        path = self.output + "0"
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        phi = (self.nw + self.beta) / (self.nk[None, :] + self.V * self.beta)
        with open(path, "w") as f:
            for k in range(self.K):
                top = np.argsort(-phi[:, k])[: self.top]
                f.write(f"{k}topic\t" + "".join(f"{self.id2word[int(w)]}:{phi[w, k]:f}|" for w in top) + "\n")


def main(cfg_file: str):
    pt = json_parser(cfg_file)
    s = gLDA_serial(pt.check_parse("input", str), pt.parse("output", str), pt.parse("alpha", float),
                    pt.parse("beta", float), pt.parse("k_topics", int), pt.parse("iters", int),
                    int(pt.get("top_words", 10)))
    s.solve()
    s.save()


if __name__ == "__main__":
    raise SystemExit(cli(main))
