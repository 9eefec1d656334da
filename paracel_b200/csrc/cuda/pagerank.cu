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
};

template <int TPR>
__global__ void __launch_bounds__(256) pagerank_pull_kernel(PrArgs a) {
  const int sub = threadIdx.x % TPR;
  const long long grp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / TPR;
  const long long ngrp = ((long long)gridDim.x * blockDim.x) / TPR;
  double dl = 0.0;
  for (long long v = grp; v < a.n_local; v += ngrp) {
    const long long b = a.row_ptr[v], e = a.row_ptr[v + 1];
    float s = 0.f;
    for (long long p = b + sub; p < e; p += TPR) s += __ldg(a.contrib + a.cols[p]);
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (sub == 0) {
      const float pr = (1.f - a.damping) + a.damping * s;
      a.new_contrib[v] = pr * a.inv_outdeg[v];
      if (a.new_rank) {
        if (a.delta_l1) dl += fabs((double)pr - (double)a.old_rank[v]);
        a.new_rank[v] = pr;
      }
    }
  }
  if (a.delta_l1 != nullptr) {
    dl = pcl_warp_sum_d(dl);
    if ((threadIdx.x & 31) == 0 && dl != 0.0) atomicAdd(a.delta_l1, dl);
  }
}

}  // namespace

PCL_API int pcl_pagerank_pull(const long long* row_ptr, const int* cols, const float* contrib,
                              const float* inv_outdeg, long long n_local, float damping,
                              float* new_contrib, float* new_rank, double* delta_l1,
                              const float* old_rank, int threads_per_row, cudaStream_t stream) {
  if (n_local <= 0) return 0;
  PrArgs a{row_ptr, cols, contrib, inv_outdeg, n_local, damping, new_contrib, new_rank, delta_l1,
           old_rank};
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
  return pcl_last_error();
}
