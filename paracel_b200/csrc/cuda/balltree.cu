// Batched maximum-inner-product search over a ball tree held in device memory
// (device form of tool/balltree/balltree.hpp:405-527: branch and bound with the
// bound  q.mu + |q| * radius  per ball, nearer child first, leaves of <= `limit`
// items scanned linearly).  One warp serves one query:
//   * the query sits in shared memory, ball bounds are warp-wide dot products;
//   * the running top-k (k <= 32) lives one entry per lane, sorted by decreasing score,
//     so the pruning threshold is a single shuffle and an insertion is one ballot
//     plus one shift;
//   * the traversal stack (node, bound) is per warp in shared memory; a query whose
//     stack would overflow is flagged (visited = -1) and left to the caller's
//     brute-force path.
// Items are stored in tree order (a leaf is a contiguous block), ids map back to the
// caller's numbering.
#include "common.cuh"

namespace {

constexpr int BT_STACK = 128;
constexpr float BT_NEG = -3.402823466e38f;

struct BtArgs {
  const int* child;        // 2 per node: left, right (-1: leaf)
  const long long* range;  // 2 per node: begin, end in tree order
  const float* radius;     // per node
  const float* mu;         // nodes x dim
  const float* items;      // n x dim, tree order
  const long long* ids;    // n original ids, tree order
  const float* queries;    // nq x dim
  int dim, nq, k;
  long long* out_idx;      // nq x k
  float* out_score;        // nq x k
  int* visited;            // nq: balls opened (-1: stack overflow)
};

__device__ __forceinline__ float warp_dot(const float* q, const float* v, int dim, int lane) {
  float s = 0.f;
  for (int d = lane; d < dim; d += 32) s = fmaf(q[d], __ldg(v + d), s);
  return pcl_warp_sum(s);
}

__global__ void __launch_bounds__(128) balltree_search_kernel(BtArgs a) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = blockIdx.x * 4 + warp;
  const int dpad = (a.dim + 3) & ~3;
  float* q = sm + warp * (dpad + 2 * BT_STACK);
  int* st_node = reinterpret_cast<int*>(q + dpad);
  float* st_bound = reinterpret_cast<float*>(st_node + BT_STACK);
  if (qi >= a.nq) return;

  float qq = 0.f;
  for (int d = lane; d < a.dim; d += 32) {
    const float v = a.queries[(long long)qi * a.dim + d];
    q[d] = v;
    qq = fmaf(v, v, qq);
  }
  __syncwarp();
  const float qn = sqrtf(pcl_warp_sum(qq));

  float best = BT_NEG;          // lane j: score of the j-th best so far
  long long best_id = -1;
  int filled = 0;
  int opened = 0;
  bool overflow = false;

  int sp = 0;
  if (lane == 0) {
    st_node[0] = 0;
    st_bound[0] = 3.402823466e38f;
  }
  sp = 1;
  __syncwarp();

  while (sp > 0) {
    --sp;
    const int id = st_node[sp];
    const float bnd = st_bound[sp];
    __syncwarp();
    const float thr = filled >= a.k ? __shfl_sync(0xffffffffu, best, a.k - 1) : BT_NEG;
    if (filled >= a.k && bnd <= thr) continue;
    ++opened;
    const int left = __ldg(a.child + 2 * id), right = __ldg(a.child + 2 * id + 1);
    if (left < 0) {
      const long long b = __ldg(a.range + 2 * id), e = __ldg(a.range + 2 * id + 1);
      for (long long t0 = b; t0 < e; t0 += 32) {
        const long long t = t0 + lane;
        float s = BT_NEG;
        long long iid = -1;
        if (t < e) {
          const float* row = a.items + t * a.dim;
          float acc = 0.f;
          for (int d = 0; d < a.dim; ++d) acc = fmaf(q[d], __ldg(row + d), acc);
          s = acc;
          iid = __ldg(a.ids + t);
        }
        unsigned m = __ballot_sync(0xffffffffu, t < e);
        while (m) {
          const int src = __ffs(m) - 1;
          m &= m - 1;
          const float cs = __shfl_sync(0xffffffffu, s, src);
          const long long cid = __shfl_sync(0xffffffffu, iid, src);
          const float th = filled >= a.k ? __shfl_sync(0xffffffffu, best, a.k - 1) : BT_NEG;
          if (filled < a.k || cs > th) {
            // sorted insert: entries that are >= cs stay in front
            const int pos = __popc(__ballot_sync(0xffffffffu, best >= cs));
            const float up = __shfl_up_sync(0xffffffffu, best, 1);
            const long long up_id = __shfl_up_sync(0xffffffffu, best_id, 1);
            if (lane > pos) { best = up; best_id = up_id; }
            else if (lane == pos) { best = cs; best_id = cid; }
            if (filled < 32) ++filled;
          }
        }
      }
    } else {
      const float bl = warp_dot(q, a.mu + (long long)left * a.dim, a.dim, lane) + qn * __ldg(a.radius + left);
      const float br = warp_dot(q, a.mu + (long long)right * a.dim, a.dim, lane) + qn * __ldg(a.radius + right);
      if (sp + 2 > BT_STACK) { overflow = true; break; }
      // the nearer (larger bound) child is pushed last, so it is opened first
      if (lane == 0) {
        if (bl >= br) {
          st_node[sp] = right; st_bound[sp] = br;
          st_node[sp + 1] = left; st_bound[sp + 1] = bl;
        } else {
          st_node[sp] = left; st_bound[sp] = bl;
          st_node[sp + 1] = right; st_bound[sp + 1] = br;
        }
      }
      sp += 2;
      __syncwarp();
    }
  }
  if (lane < a.k) {
    a.out_idx[(long long)qi * a.k + lane] = lane < filled ? best_id : -1;
    a.out_score[(long long)qi * a.k + lane] = lane < filled ? best : BT_NEG;
  }
  if (lane == 0 && a.visited != nullptr) a.visited[qi] = overflow ? -1 : opened;
}

}  // namespace

// Top-k (1 <= k <= 32) inner products of `nq` queries against the items of a ball tree.
// Arrays as exported by the host tree: child [2 * nodes], range [2 * nodes] (positions in
// tree order), radius [nodes], mu [nodes x dim], items [n x dim] in tree order, ids [n].
// out_idx / out_score are nq x k, best first (-1 / -FLT_MAX where fewer than k items exist);
// visited[q] is the number of balls opened, or -1 if the traversal stack overflowed.
PCL_API int pcl_balltree_search(const int* child, const long long* range, const float* radius,
                                const float* mu, const float* items, const long long* ids,
                                const float* queries, int dim, int nq, int k, long long* out_idx,
                                float* out_score, int* visited, cudaStream_t stream) {
  if (nq <= 0) return 0;
  if (k < 1 || k > 32 || dim < 1) return (int)cudaErrorInvalidValue;
  BtArgs a{child, range, radius, mu, items, ids, queries, dim, nq, k, out_idx, out_score, visited};
  const int dpad = (dim + 3) & ~3;
  const size_t smem = 4 * (size_t)(dpad + 2 * BT_STACK) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(balltree_search_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  balltree_search_kernel<<<(nq + 3) / 4, 128, smem, stream>>>(a);
  return pcl_last_error();
}
