// Collapsed Gibbs sampling for LDA, one warp per document.
//
// Sampler (reference: alg/topic_model/gLDA.hpp:408-426 and 396-406): remove the token,
//   p(k) ~ (n_dk + alpha) / (n_d + K alpha) * (n_wk + beta) / (n_k + V beta),
// draw k by inverse CDF, add the token back.  The document factor's denominator does not
// depend on k and is dropped.
//
// Mapping: K = 128 * J topics; lane l keeps topics {128 j + 4 l + t} (j < J, t < 4), i.e. its
// part of a word row is J coalesced 128-bit loads.  The document's topic counts live in
// registers for the whole document (exact within a document, like the sequential sweep);
// word-topic rows and topic sums are this rank's working copies of the parameter-server
// rows and are updated with integer atomics, so concurrent documents never lose counts
// (AD-LDA: counts of other documents may be slightly stale).  1 / (n_k + V beta) is read
// once per document.  The push of (current - snapshot) to the owners happens afterwards
// with rows_push_i32.
//
// Measured and not kept: requesting the next token's word-topic row before the current token is
// sampled (software pipelining of the L2 latency).  The second row costs 32 more registers
// (162 instead of 128 at K = 1024), residency drops from 16 to 12 warps per SM and the
// sampler went from 1.33 G to 0.84 G tokens/s on the 1 M-document configuration.
// Kept: 1 / (n_k + V beta) in shared memory instead of registers (128 -> 95 registers, 16 -> 20
// warps per SM, 1.32 G -> 1.41 G tokens/s).  Parking the lane's running sums there as well (80
// registers, 24 warps, 32 KB of shared memory per block) was slower again: 1.36 G.
// Also measured and not kept: a prefetch.global.L2 of the next token's row (no registers held):
// 1.26 G tokens/s against 1.41 G.
#include "common.cuh"

namespace {

struct LdaArgs {
  const long long* doc_ptr;  // n_docs + 1
  const int* words;          // local word index per token
  int* z;                    // topic per token (in/out)
  int* n_dk;                 // n_docs x K (in/out)
  int* n_wk;                 // n_local_words x K working copy (atomics)
  int* n_k;                  // K working copy (atomics)
  long long n_docs;
  float alpha, beta, vbeta;
  unsigned long long seed;
};

__device__ __forceinline__ float u01(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ULL;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
  x ^= x >> 31;
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

template <int J>
__global__ void __launch_bounds__(128) lda_gibbs_kernel(LdaArgs a) {
  constexpr int K = 128 * J;
  constexpr int R = 4 * J;  // topics per lane
  // 1 / (n_k + V beta) of the lane's topics lives in shared memory, not in registers: the lane
  // writes its R values at the start of a document and reads them back (J 128-bit loads) for every
  // token.  At K = 1024 this takes the kernel from 128 to about 96 registers, i.e. from 16 to 20
  // resident warps per SM, which matters because the sampler is bound by latency.
  __shared__ float4 s_inv[4][J][32];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long d = warp; d < a.n_docs; d += nwarps) {
    const long long t0 = a.doc_ptr[d], t1 = a.doc_ptr[d + 1];
    if (t1 <= t0) continue;
    int nd[R];
    int* ndp = a.n_dk + d * K;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int4 v = *reinterpret_cast<const int4*>(ndp + 128 * j + 4 * lane);
      nd[4 * j] = v.x; nd[4 * j + 1] = v.y; nd[4 * j + 2] = v.z; nd[4 * j + 3] = v.w;
      const int4 s = __ldcg(reinterpret_cast<const int4*>(a.n_k + 128 * j + 4 * lane));
      s_inv[wib][j][lane] = make_float4(1.f / ((float)s.x + a.vbeta), 1.f / ((float)s.y + a.vbeta),
                                        1.f / ((float)s.z + a.vbeta), 1.f / ((float)s.w + a.vbeta));
    }
    for (long long t = t0; t < t1; ++t) {
      const int w = __ldg(a.words + t);
      const int k_old = a.z[t];
      int* nwp = a.n_wk + (long long)w * K;
      // remove the token
      const int lo = (k_old & 127) >> 2, ro = ((k_old >> 7) << 2) | (k_old & 3);
      if (lane == lo) {
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r == ro) nd[r] -= 1;
        atomicSub(nwp + k_old, 1);
        atomicSub(a.n_k + k_old, 1);
      }
      __syncwarp();
      // unnormalised posterior, running sums inside the lane
      float p[R];
      float run = 0.f;
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const int4 v = __ldcg(reinterpret_cast<const int4*>(nwp + 128 * j + 4 * lane));
        const int c[4] = {v.x, v.y, v.z, v.w};
        const float4 iv4 = s_inv[wib][j][lane];
        const float iv[4] = {iv4.x, iv4.y, iv4.z, iv4.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int r = 4 * j + q;
          // a concurrent document may have pushed a count of this word below zero transiently
          const float nw = fmaxf((float)c[q], 0.f);
          run += ((float)nd[r] + a.alpha) * (nw + a.beta) * iv[q];
          p[r] = run;
        }
      }
      // warp scan of the lane totals
      float incl = run;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      const float total = __shfl_sync(0xffffffffu, incl, 31);
      const float x = u01(a.seed ^ ((unsigned long long)t * 0x9E3779B1ULL + (unsigned long long)d)) * total;
      const unsigned ball = __ballot_sync(0xffffffffu, incl > x);
      const int sel = ball ? (__ffs(ball) - 1) : 31;
      int k_new = 0;
      if (lane == sel) {
        const float base = incl - run;
        int r_sel = R - 1;
#pragma unroll
        for (int r = R - 1; r >= 0; --r)
          if (base + p[r] > x) r_sel = r;
        k_new = ((r_sel >> 2) << 7) + 4 * lane + (r_sel & 3);
#pragma unroll
        for (int r = 0; r < R; ++r)
          if (r == r_sel) nd[r] += 1;
        atomicAdd(nwp + k_new, 1);
        atomicAdd(a.n_k + k_new, 1);
        a.z[t] = k_new;
      }
      __syncwarp();
    }
#pragma unroll
    for (int j = 0; j < J; ++j)
      *reinterpret_cast<int4*>(ndp + 128 * j + 4 * lane) =
          make_int4(nd[4 * j], nd[4 * j + 1], nd[4 * j + 2], nd[4 * j + 3]);
  }
}

struct LlArgs {
  const long long* doc_ptr;
  const int* words;
  const int* n_dk;
  const int* n_wk;
  const int* n_k;
  const int* doc_len;
  long long n_docs;
  int K;
  float alpha, beta, vbeta;
  double* out;
};

// sum over tokens of log sum_k theta_dk phi_kw  (gLDA.hpp:447-463)
__global__ void __launch_bounds__(128) lda_loglik_kernel(LlArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  double acc = 0.0;
  for (long long d = warp; d < a.n_docs; d += nwarps) {
    const float den = (float)a.doc_len[d] + a.K * a.alpha;
    for (long long t = a.doc_ptr[d]; t < a.doc_ptr[d + 1]; ++t) {
      const int* nwp = a.n_wk + (long long)a.words[t] * a.K;
      float s = 0.f;
      for (int k = lane; k < a.K; k += 32)
        s += ((float)a.n_dk[d * a.K + k] + a.alpha) / den * (fmaxf((float)nwp[k], 0.f) + a.beta) /
             ((float)a.n_k[k] + a.vbeta);
      s = pcl_warp_sum(s);
      acc += (double)__logf(s + 1e-30f);
    }
  }
  if (lane == 0 && acc != 0.0) atomicAdd(a.out, acc);
}

}  // namespace

// One Gibbs sweep over `n_docs` documents.  K must be 128, 256, 512 or 1024.
PCL_API int pcl_lda_gibbs(const long long* doc_ptr, const int* words, int* z, int* n_dk, int* n_wk,
                          int* n_k, long long n_docs, int K, float alpha, float beta, float vbeta,
                          unsigned long long seed, int blocks, cudaStream_t stream) {
  if (n_docs <= 0) return 0;
  LdaArgs a{doc_ptr, words, z, n_dk, n_wk, n_k, n_docs, alpha, beta, vbeta, seed};
  // default grid: as many blocks as fit on the device at once (the warps loop over the documents)
#define PCL_LDA_LAUNCH(JJ)                                                                          \
  {                                                                                                 \
    if (blocks <= 0) {                                                                              \
      int per_sm = 0;                                                                               \
      cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lda_gibbs_kernel<JJ>, 128, 0); \
      if (e != cudaSuccess) return (int)e;                                                          \
      blocks = 148 * (per_sm > 0 ? per_sm : 4);                                                     \
    }                                                                                               \
    const long long need = (n_docs + 3) / 4;                                                        \
    if (need < blocks) blocks = (int)need;                                                          \
    lda_gibbs_kernel<JJ><<<blocks, 128, 0, stream>>>(a);                                            \
  }
  switch (K) {
    case 128: PCL_LDA_LAUNCH(1) break;
    case 256: PCL_LDA_LAUNCH(2) break;
    case 512: PCL_LDA_LAUNCH(4) break;
    case 1024: PCL_LDA_LAUNCH(8) break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef PCL_LDA_LAUNCH
  return pcl_last_error();
}

PCL_API int pcl_lda_loglik(const long long* doc_ptr, const int* words, const int* n_dk, const int* n_wk,
                           const int* n_k, const int* doc_len, long long n_docs, int K, float alpha,
                           float beta, float vbeta, double* out, cudaStream_t stream) {
  if (n_docs <= 0) return 0;
  LlArgs a{doc_ptr, words, n_dk, n_wk, n_k, doc_len, n_docs, K, alpha, beta, vbeta, out};
  long long need = (n_docs + 3) / 4;
  int blocks = need < 148 * 8 ? (int)need : 148 * 8;
  lda_loglik_kernel<<<blocks, 128, 0, stream>>>(a);
  return pcl_last_error();
}
