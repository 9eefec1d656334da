"""LDA by collapsed Gibbs sampling with delta pushes (AD-LDA style; reference:
alg/topic_model/gLDA.hpp:40-500, gLDA_driver.cpp; serial version tool/gLDA_serial.cpp).

Host path: the global dictionary is built through the server (``gLDA_dict_update``), topic
assignments start uniform at random, and one iteration is a sequential sweep over the local
tokens with ``p(k) ~ (n_dk + alpha)/(n_d + K alpha) * (n_wk + beta)/(n_k + V beta)`` and
inverse-CDF sampling, followed by a push of the deltas of the local word rows and topic
sums, a barrier and a fresh pull (gLDA.hpp:408-445).

Device path (``lda_gpu.LdaGibbsGpu``): word-topic counts are an int32 ``RowTable`` in HBM,
one warp samples one document with its doc-topic counts in registers
(``csrc/cuda/lda.cu``), word rows are pulled / pushed sparsely per minibatch with SSP."""
from __future__ import annotations

import math
import os
import time
from typing import Dict, List

import numpy as np

from .._core import core
from ..paralg import paralg


class LDAmodel(paralg):
    def __init__(self, comm, hosts_dct_str, input: str, output: str = "", alpha: float = 0.1,
                 beta: float = 0.1, k_topics: int = 10, iters: int = 10, top_words: int = 10,
                 handle_file: str = "", debug: bool = False, seed: int = 0, **kw):
        super().__init__(hosts_dct_str, comm, "", iters, **kw)
        self.input, self.out_prefix = input, output
        self.alpha, self.beta, self.K = float(alpha), float(beta), int(k_topics)
        self.max_iter, self.top, self.handle_fn, self.debug = int(iters), int(top_words), handle_file, debug
        self.seed = seed
        self.worker_id = self.get_worker_id()
        self.compute = self.update = 0.0
        self.loglik: List[float] = []

    # ----------------------------------------------------------------- load
    def load(self):
        lines = [l for l in self.paracel_load(self.input)]
        docs_tok = [l.split() for l in lines]
        local_words: Dict[str, int] = {}
        for toks in docs_tok:
            for w in toks:
                if w not in local_words:
                    local_words[w] = len(local_words)
        self.paracel_bupdate("global_dict", local_words, self.handle_fn, "gLDA_dict_update")
        self.paracel_sync()
        self.word2id = {w: int(i) for w, i in self.paracel_read("global_dict").items()}
        self.V = len(self.word2id)
        self.id2word = {i: w for w, i in self.word2id.items()}
        gids = sorted({self.word2id[w] for w in local_words})
        self.local_vocab = np.asarray(gids, dtype=np.int64)
        pos = {g: j for j, g in enumerate(gids)}
        self.local_dict_list = [str(g) for g in gids]
        lens = [len(t) for t in docs_tok]
        self.M = len(docs_tok)
        self.doc_ptr = np.zeros(self.M + 1, dtype=np.int64)
        np.cumsum(lens, out=self.doc_ptr[1:])
        self.T = int(self.doc_ptr[-1])
        self.words = np.fromiter((pos[self.word2id[w]] for t in docs_tok for w in t), dtype=np.int32,
                                 count=self.T)
        self.doc_len = np.asarray(lens, dtype=np.int32)

    def para_init(self):
        K = self.K
        rng = np.random.default_rng(self.seed + 10 * self.worker_id)
        self.z = rng.integers(0, K, size=self.T, dtype=np.int32)
        self.doc_topic = np.zeros((self.M, K), dtype=np.int32)
        doc_of = np.repeat(np.arange(self.M), self.doc_len)
        np.add.at(self.doc_topic, (doc_of, self.z), 1)
        self.word_topic = np.zeros((self.local_vocab.size, K), dtype=np.int32)
        np.add.at(self.word_topic, (self.words, self.z), 1)
        self.topic_sum = np.bincount(self.z, minlength=K).astype(np.int32)
        self.global_topic_key = [f"sum_topic_{k}" for k in range(K)]
        self.last_word_topic = np.zeros_like(self.word_topic)
        self.last_topic_sum = np.zeros_like(self.topic_sum)
        self._exchange()
        self.paracel_sync()

    def _exchange(self):
        """Push deltas since the last exchange, barrier, pull the fresh global counts."""
        dw = self.word_topic - self.last_word_topic
        ds = self.topic_sum - self.last_topic_sum
        if self.local_dict_list:
            self.paracel_bupdate_multi(self.local_dict_list, dw.tolist(), self.handle_fn,
                                       "gLDA_word_update")
        self.paracel_bupdate_multi(self.global_topic_key, ds.tolist(), self.handle_fn,
                                   "gLDA_sum_topic_update")
        self.paracel_sync()
        if self.local_dict_list:
            self.word_topic = np.ascontiguousarray(
                np.asarray(self.paracel_read_multi(self.local_dict_list), dtype=np.int32))
        self.topic_sum = np.asarray(self.paracel_read_multi(self.global_topic_key), dtype=np.int32)
        self.last_word_topic = self.word_topic.copy()
        self.last_topic_sum = self.topic_sum.copy()

    # ---------------------------------------------------------------- train
    def single_iter(self, it: int = 0):
        t0 = time.time()
        core().lda_gibbs_sweep(self.doc_ptr, self.words, self.z, self.doc_topic, self.word_topic,
                               self.topic_sum, self.doc_len, self.K, self.V, self.alpha, self.beta,
                               (self.seed * 1000003 + it * 131 + self.worker_id) & 0xFFFFFFFFFFFF)
        self.compute += time.time() - t0
        t0 = time.time()
        self._exchange()
        self.update += time.time() - t0

    def train(self):
        for i in range(self.max_iter):
            self.single_iter(i)
            if self.debug:
                self.loglik.append(self.likelihood())

    def likelihood(self) -> float:
        """Sum over tokens of log sum_k theta_dk phi_kw, all-reduced (gLDA.hpp:447-463)."""
        K = self.K
        theta = (self.doc_topic + self.alpha) / (self.doc_len[:, None] + K * self.alpha)
        phi = (self.word_topic + self.beta) / (self.topic_sum[None, :] + self.V * self.beta)
        doc_of = np.repeat(np.arange(self.M), self.doc_len)
        s = 0.0
        step = 1 << 16
        for b in range(0, self.T, step):
            p = (theta[doc_of[b:b + step]] * phi[self.words[b:b + step]]).sum(1)
            s += float(np.log(p + 1e-300).sum())
        return self.worker_comm.allreduce(s)

    def perplexity(self) -> float:
        T = self.worker_comm.allreduce(int(self.T))
        return math.exp(-self.likelihood() / max(T, 1))

    def solve(self):
        self.load()
        self.para_init()
        self.train()

    def save(self):
        """Top words per topic, one line ``<k>topic\\t<word>:<p>|...|`` in ``<output><rank>``;
        topic k is written by worker k % W after a shuffle through the server."""
        self.paracel_sync()
        Vb = self.V * self.beta
        dump_phi = {}
        for j in range(self.K):
            col = self.word_topic[:, j]
            nz = np.nonzero(col)[0]
            for li in nz:
                dump_phi[f"key_{j}_{self.local_vocab[li]}"] = float(
                    (col[li] + self.beta) / (self.topic_sum[j] + Vb))
            if j % 5 == 0 or j == self.K - 1:
                if dump_phi:
                    self.paracel_write_multi(dump_phi)
                dump_phi = {}
        self.paracel_sync()
        W, me = self.get_worker_size(), self.worker_id
        dump_data: Dict[int, list] = {}

        def parse(d):
            for key, p in d.items():
                _, tid, wid = key.split("_")
                tid = int(tid)
                if tid % W != me:
                    continue
                dump_data.setdefault(tid, []).append((int(wid), p))
        self.paracel_read_special_handle(self.handle_fn, "gLDA_dump_filter", parse)
        path = self.out_prefix + str(me)
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(path, "w") as f:
            for tid in sorted(dump_data):
                vals = sorted(dump_data[tid], key=lambda x: -x[1])[: self.top]
                f.write(f"{tid}topic\t" + "".join(f"{self.id2word[w]}:{p:f}|" for w, p in vals) + "\n")
        self.paracel_sync()
