// PageRank pull step over the in-link CSR of this rank's vertices:
//   pr(v) = (1 - d) + d * sum_{u -> v} pr(u) / outdeg(u)
// (reference: alg/graph_alg/pagerank/pr.hpp:154-160; ranks are not re-normalised and
// start at 1/N, pr.hpp:109-118).  `contrib[u]` = pr(u) / outdeg(u) is the full vector that
// dense_read gathered from all owners; the kernel writes the new contribution of every
// local vertex straight into this rank's shard of that vector (the "write_multi" of
// pr.hpp:163-168) and optionally the plain rank.  A group of TPR threads handles one row.
#include "common.cuh"

namespace {

struct PrArgs {
  const long long* row_ptr;   // n_local + 1 (in-links)
  const int* cols;            // global ids of the in-neighbours
  const float* contrib;       // full gathered vector
  const float* inv_outdeg;    // n_local: 1 / outdeg(v), 0 for vertices without out-links
  long long n_local;
  float damping;
  float* new_contrib;         // n_local (this rank's shard of the contribution vector)
  float* new_rank;            // n_local, may be null
  double* delta_l1;           // optional: += sum |new - old| of the local ranks
  const float* old_rank;      // needed when delta_l1 is given
  long long heavy_deg;        // rows with more in-links than this are left to the heavy kernel
  const int* heavy_rows;      // list of those rows
  int n_heavy;
};

template <int TPR>
__global__ void __launch_bounds__(256) pagerank_pull_kernel(PrArgs a) {
  const int sub = threadIdx.x % TPR;
  const long long grp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / TPR;
  const long long ngrp = ((long long)gridDim.x * blockDim.x) / TPR;
  // groups of one warp run different numbers of iterations: shuffle only within the group
  const unsigned gmask = TPR == 32 ? 0xffffffffu
                                   : (((1u << TPR) - 1u) << ((threadIdx.x & 31) - sub));
  double dl = 0.0;
  for (long long v = grp; v < a.n_local; v += ngrp) {
    const long long b = a.row_ptr[v], e = a.row_ptr[v + 1];
    if (e - b > a.heavy_deg) continue;  // uniform within the group
    float s = 0.f;
    for (long long p = b + sub; p < e; p += TPR) s += __ldg(a.contrib + a.cols[p]);
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(gmask, s, o);
    if (sub == 0) {
      const float pr = (1.f - a.damping) + a.damping * s;
      a.new_contrib[v] = pr * a.inv_outdeg[v];
      if (a.new_rank) {
        if (a.delta_l1) dl += fabs((double)pr - (double)a.old_rank[v]);
        a.new_rank[v] = pr;
      }
    }
  }
  __syncwarp();
  if (a.delta_l1 != nullptr) {
    dl = pcl_warp_sum_d(dl);
    if ((threadIdx.x & 31) == 0 && dl != 0.0) atomicAdd(a.delta_l1, dl);
  }
}

// Rows with very many in-links (power-law graphs have a few with hundreds of thousands):
// one CTA per row, block-wide reduction.
__global__ void __launch_bounds__(256) pagerank_heavy_kernel(PrArgs a) {
  __shared__ float red[8];
  for (int h = blockIdx.x; h < a.n_heavy; h += gridDim.x) {
    const int v = a.heavy_rows[h];
    const long long b = a.row_ptr[v], e = a.row_ptr[v + 1];
    float s = 0.f;
    for (long long p = b + threadIdx.x; p < e; p += blockDim.x) s += __ldg(a.contrib + a.cols[p]);
    s = pcl_warp_sum(s);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
      const float pr = (1.f - a.damping) + a.damping * t;
      a.new_contrib[v] = pr * a.inv_outdeg[v];
      if (a.new_rank) {
        if (a.delta_l1) atomicAdd(a.delta_l1, fabs((double)pr - (double)a.old_rank[v]));
        a.new_rank[v] = pr;
      }
    }
  }
}

// Edge-balanced variant ("CSR stream"): a block owns PR_CAP consecutive in-links whatever rows
// they belong to.  The neighbours' contributions are gathered into shared memory with fully
// coalesced index reads, then one warp per row sums the row's segment.  A row that lies
// completely inside the block is stored, a row cut by a block boundary (including rows far
// longer than a block) is accumulated with atomicAdd, so `acc` must be zero on entry.  The
// damping epilogue is a second, element-wise kernel because a cut row is only complete once
// all its blocks have run.
// PR_CAP is 2048 or 4096 in-links per block (template parameter).  Which is faster depends on the
// graph's labelling (R-MAT 26, one GPU: raw labels 6.28 ms with 2048 and 6.04 ms with 4096;
// block-scrambled labels 7.74 ms and 8.97 ms), so the model times both once at load time.
constexpr int PR_ROWS = 1024;   // row pointers of a block cached in shared memory up to this many rows

// blk_first[b] / blk_last[b]: the rows that contain in-link b * PR_CAP and the last in-link of
// block b (static per graph, computed once at load time).
template <int PR_CAP>
__global__ void __launch_bounds__(256) pagerank_stream_kernel(const long long* row_ptr, const int* cols,
                                                              const float* contrib,
                                                              const int* blk_first, const int* blk_last,
                                                              long long nnz, float* acc) {
  __shared__ float sv[PR_CAP];
  __shared__ int srp[PR_ROWS + 1];   // row pointers relative to the block start, clamped to [0, len]
  __shared__ int long_rows[64];
  __shared__ int n_long;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long blk = blockIdx.x; blk * PR_CAP < nnz; blk += gridDim.x) {
    const long long s = blk * PR_CAP;
    const long long e = (s + PR_CAP < nnz) ? s + PR_CAP : nnz;
    const int len = (int)(e - s);
    const long long r0 = blk_first[blk], r1 = blk_last[blk];
    const long long nrows = r1 - r0 + 1;
    __syncthreads();
    if (threadIdx.x == 0) n_long = 0;
    // all index loads of the thread first, then all gathers, then the stores: eight independent
    // random reads in flight per thread instead of a load-use chain per element
#pragma unroll
    for (int h = 0; h < PR_CAP / 2048; ++h) {   // batches of eight gathers per thread
      int ci[8];
      float cv[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const long long p = s + threadIdx.x + (h * 8 + q) * 256;
        ci[q] = p < e ? __ldg(cols + p) : -1;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) cv[q] = ci[q] >= 0 ? __ldg(contrib + ci[q]) : 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (ci[q] >= 0) sv[threadIdx.x + (h * 8 + q) * 256] = cv[q];
    }
    const bool cached = nrows <= PR_ROWS;
    if (cached) {
      for (int i = threadIdx.x; i <= (int)nrows; i += blockDim.x) {
        long long v = row_ptr[r0 + i] - s;
        srp[i] = v < 0 ? 0 : (v > len ? len : (int)v);
      }
    }
    __syncthreads();
    // phase A: one thread per row for short segments
    for (long long i = threadIdx.x; i < nrows; i += blockDim.x) {
      int b, en;
      if (cached) { b = srp[i]; en = srp[i + 1]; }
      else {
        long long vb = row_ptr[r0 + i] - s, ve = row_ptr[r0 + i + 1] - s;
        b = vb < 0 ? 0 : (int)vb;
        en = ve > len ? len : (int)ve;
      }
      const int cnt = en - b;
      if (cnt <= 0) continue;
      if (cnt > 64) {
        const int slot = atomicAdd(&n_long, 1);
        if (slot < 64) { long_rows[slot] = (int)i; continue; }
      }
      float sum = 0.f;
      for (int p = b; p < en; ++p) sum += sv[p];
      const long long r = r0 + i;
      const bool whole = (i > 0 || row_ptr[r] >= s) && (i < nrows - 1 || row_ptr[r + 1] <= e);
      if (whole) acc[r] = sum;
      else atomicAdd(acc + r, sum);
    }
    __syncthreads();
    // phase B: a warp per long segment
    const int nl = n_long < 64 ? n_long : 64;
    for (int q = warp; q < nl; q += 8) {
      const long long i = long_rows[q];
      const long long r = r0 + i;
      const long long rb = row_ptr[r], re = row_ptr[r + 1];
      const int b = rb > s ? (int)(rb - s) : 0, en = re < e ? (int)(re - s) : len;
      float sum = 0.f;
      for (int p = b + lane; p < en; p += 32) sum += sv[p];
      sum = pcl_warp_sum(sum);
      if (lane == 0) {
        if (rb >= s && re <= e) acc[r] = sum;
        else atomicAdd(acc + r, sum);
      }
    }
  }
}

__global__ void __launch_bounds__(256) pagerank_epilogue_kernel(PrArgs a, const float* acc) {
  double dl = 0.0;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < a.n_local;
       v += (long long)gridDim.x * blockDim.x) {
    const float pr = (1.f - a.damping) + a.damping * acc[v];
    a.new_contrib[v] = pr * a.inv_outdeg[v];
    if (a.new_rank) {
      if (a.delta_l1) dl += fabs((double)pr - (double)a.old_rank[v]);
      a.new_rank[v] = pr;
    }
  }
  if (a.delta_l1 != nullptr) {
    dl = pcl_warp_sum_d(dl);
    if ((threadIdx.x & 31) == 0 && dl != 0.0) atomicAdd(a.delta_l1, dl);
  }
}

}  // namespace

// Edge-balanced pull step.  `acc` is a scratch vector of n_local floats; it is cleared here.
// blk_first / blk_last have ceil(nnz / cap) entries (see pagerank_stream_kernel); cap is 2048 or 4096.
PCL_API int pcl_pagerank_pull_stream(const long long* row_ptr, const int* cols, const float* contrib,
                                     const float* inv_outdeg, long long n_local, long long nnz,
                                     const int* blk_first, const int* blk_last, float damping, float* acc, float* new_contrib, float* new_rank,
                                     double* delta_l1, const float* old_rank, int cap, cudaStream_t stream) {
  if (n_local <= 0) return 0;
  if (cap != 2048 && cap != 4096) return (int)cudaErrorInvalidValue;
  if (delta_l1 != nullptr && (old_rank == nullptr || new_rank == nullptr)) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(acc, 0, (size_t)n_local * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  if (nnz > 0) {
    long long blocks = (nnz + cap - 1) / cap;
    if (blocks > 148LL * 64) blocks = 148LL * 64;
    if (cap == 2048)
      pagerank_stream_kernel<2048><<<(int)blocks, 256, 0, stream>>>(row_ptr, cols, contrib, blk_first, blk_last, nnz, acc);
    else
      pagerank_stream_kernel<4096><<<(int)blocks, 256, 0, stream>>>(row_ptr, cols, contrib, blk_first, blk_last, nnz, acc);
  }
  PrArgs a{row_ptr, cols, contrib, inv_outdeg, n_local, damping, new_contrib, new_rank, delta_l1,
           old_rank, 0, nullptr, 0};
  long long eb = (n_local + 255) / 256;
  if (eb > 148 * 16) eb = 148 * 16;
  pagerank_epilogue_kernel<<<(int)eb, 256, 0, stream>>>(a, acc);
  return pcl_last_error();
}

PCL_API int pcl_pagerank_pull(const long long* row_ptr, const int* cols, const float* contrib,
                              const float* inv_outdeg, long long n_local, float damping,
                              float* new_contrib, float* new_rank, double* delta_l1,
                              const float* old_rank, int threads_per_row, long long heavy_deg,
                              const int* heavy_rows, int n_heavy, cudaStream_t stream) {
  if (n_local <= 0) return 0;
  if (heavy_rows == nullptr || n_heavy <= 0) { heavy_deg = 0x7fffffffffffffffLL; n_heavy = 0; }
  PrArgs a{row_ptr, cols, contrib, inv_outdeg, n_local, damping, new_contrib, new_rank, delta_l1,
           old_rank, heavy_deg, heavy_rows, n_heavy};
  if (delta_l1 != nullptr && (old_rank == nullptr || new_rank == nullptr)) return (int)cudaErrorInvalidValue;
  const int tpr = threads_per_row > 0 ? threads_per_row : 8;
  long long blocks = (n_local * tpr + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  switch (tpr) {
    case 4: pagerank_pull_kernel<4><<<(int)blocks, 256, 0, stream>>>(a); break;
    case 8: pagerank_pull_kernel<8><<<(int)blocks, 256, 0, stream>>>(a); break;
    case 16: pagerank_pull_kernel<16><<<(int)blocks, 256, 0, stream>>>(a); break;
    case 32: pagerank_pull_kernel<32><<<(int)blocks, 256, 0, stream>>>(a); break;
    default: return (int)cudaErrorInvalidValue;
  }
  if (n_heavy > 0) {
    int hb = n_heavy < 148 * 8 ? n_heavy : 148 * 8;
    pagerank_heavy_kernel<<<hb, 256, 0, stream>>>(a);
  }
  return pcl_last_error();
}
