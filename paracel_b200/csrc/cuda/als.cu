// Batched ALS normal equations: for every user u with rated items I_u and ratings a_u,
//   w_u = (H_u^T H_u + lambda I)^-1 H_u^T a_u
// (reference: alg/recommendation/als/als.hpp:133-165, which forms the k x k matrix with Eigen
// and multiplies by its explicit inverse).  Here one CTA of 256 threads handles one work
// item = one segment of a user's ratings: the 16 x 16 thread grid keeps the k x k Gram
// matrix in registers ((k/16)^2 per thread), item rows are staged through shared memory 8 at
// a time, and the system is solved in shared memory by a blocked Cholesky factorisation
// (16-column panels) and two blocked triangular solves.  Users with more ratings than one segment holds are split: every
// segment adds its partial Gram matrix and right-hand side into a scratch slot with atomics
// and the segment that arrives last solves.
//
// Where the time goes (200 k users, rank 128, CUDA events): 48 ms with 8 ratings per user, 69 ms
// with 100, 138 ms with 400, i.e. about 46 ms for the 200 k factorisations and triangular solves
// and 23 ms per 100 ratings for the Gram matrices.  The factorisation is a chain of dependent
// steps per system (16-column panels, the diagonal block by one warp), and three systems per SM
// is what the 66 KB matrix in shared memory allows; prefetching the next eight item rows under
// the products of the current eight took 4 % off the Gram part.
#include "common.cuh"

namespace {

struct AlsArgs {
  const int* seg_user;         // n_seg: user index of the segment
  const long long* seg_begin;  // n_seg: first rating (index into item_idx / rating)
  const long long* seg_end;    // n_seg
  const int* user_nseg;        // n_users: number of segments of the user
  const int* user_slot;        // n_users: scratch slot for split users, -1 otherwise
  const int* item_idx;         // nnz: row of H
  const float* rating;         // nnz
  const float* H;              // n_items x k
  float* W;                    // n_users x k (output)
  float* scratch;              // n_slots x (k*k + k), zero-initialised
  unsigned int* slot_count;    // n_slots, zero-initialised
  long long n_seg;
  int k;
  float lambda;
};

template <int KB>
__global__ void __launch_bounds__(256, 3) als_kernel(AlsArgs a) {
  constexpr int K = 16 * KB;
  extern __shared__ float sm[];
  float* sA = sm;                       // K x (K + 1)
  float* sb = sA + K * (K + 1);         // K
  float* sh = sb + K;                   // 8 x K staged item rows
  float* sr = sh + 8 * K;               // 8 ratings
  __shared__ int s_last;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (long long seg = blockIdx.x; seg < a.n_seg; seg += gridDim.x) {
    const int u = a.seg_user[seg];
    const long long b0 = a.seg_begin[seg], b1 = a.seg_end[seg];
    float acc[KB][KB];
#pragma unroll
    for (int i = 0; i < KB; ++i)
#pragma unroll
      for (int j = 0; j < KB; ++j) acc[i][j] = 0.f;
    float bacc = 0.f;  // threads 0..K-1 own one entry of H^T a
    // Eight item rows are staged per step.  The rows of step s + 1 are requested (index, then the
    // row itself: two dependent global loads) before the products of step s are formed, so that
    // latency runs under the arithmetic instead of in front of it.
    constexpr int PF = KB / 2;            // staged elements per thread and step: 8 K / 256
    float pre[PF];
    float pre_r = 0.f;
    auto fetch = [&](long long p) {
      const int cnt = (int)((b1 - p) < 8 ? (b1 - p) : 8);
#pragma unroll
      for (int q = 0; q < PF; ++q) {
        const int e = tid + q * 256;
        const int r = e / K, c = e % K;
        pre[q] = (r < cnt && c < a.k) ? __ldg(a.H + (long long)a.item_idx[p + r] * a.k + c) : 0.f;
      }
      pre_r = tid < cnt ? a.rating[p + tid] : 0.f;
    };
    if (b0 < b1) fetch(b0);
    for (long long p = b0; p < b1; p += 8) {
      const int cnt = (int)((b1 - p) < 8 ? (b1 - p) : 8);
      __syncthreads();
#pragma unroll
      for (int q = 0; q < PF; ++q) sh[tid + q * 256] = pre[q];
      if (tid < 8) sr[tid] = pre_r;
      __syncthreads();
      if (p + 8 < b1) fetch(p + 8);
      for (int r = 0; r < cnt; ++r) {
        float hy[KB], hx[KB];
        if constexpr ((KB & 3) == 0) {
#pragma unroll
          for (int i = 0; i < KB; i += 4) {
            const float4 y4 = *reinterpret_cast<const float4*>(sh + r * K + ty * KB + i);
            const float4 x4 = *reinterpret_cast<const float4*>(sh + r * K + tx * KB + i);
            hy[i] = y4.x; hy[i + 1] = y4.y; hy[i + 2] = y4.z; hy[i + 3] = y4.w;
            hx[i] = x4.x; hx[i + 1] = x4.y; hx[i + 2] = x4.z; hx[i + 3] = x4.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < KB; i += 2) {
            const float2 y2 = *reinterpret_cast<const float2*>(sh + r * K + ty * KB + i);
            const float2 x2 = *reinterpret_cast<const float2*>(sh + r * K + tx * KB + i);
            hy[i] = y2.x; hy[i + 1] = y2.y;
            hx[i] = x2.x; hx[i + 1] = x2.y;
          }
        }
#pragma unroll
        for (int i = 0; i < KB; ++i)
#pragma unroll
          for (int j = 0; j < KB; ++j) acc[i][j] = fmaf(hy[i], hx[j], acc[i][j]);
        if (tid < K) bacc = fmaf(sr[r], sh[r * K + tid], bacc);
      }
    }
    const int slot = a.user_slot[u];
    bool solve_here = true;
    if (slot >= 0) {
      // split user: add the partial sums, the last segment to arrive solves
      float* gA = a.scratch + (long long)slot * (K * K + K);
#pragma unroll
      for (int i = 0; i < KB; ++i)
#pragma unroll
        for (int j = 0; j < KB; ++j) atomicAdd(gA + (ty * KB + i) * K + tx * KB + j, acc[i][j]);
      if (tid < K) atomicAdd(gA + K * K + tid, bacc);
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const unsigned int prev = atomicAdd(a.slot_count + slot, 1u);
        s_last = (prev == (unsigned int)a.user_nseg[u] - 1) ? 1 : 0;
      }
      __syncthreads();
      solve_here = (s_last != 0);
      if (solve_here) {
        __threadfence();
#pragma unroll
        for (int i = 0; i < KB; ++i)
#pragma unroll
          for (int j = 0; j < KB; ++j) acc[i][j] = __ldcg(gA + (ty * KB + i) * K + tx * KB + j);
        if (tid < K) bacc = __ldcg(gA + K * K + tid);
      }
    }
    if (!solve_here) continue;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < KB; ++i)
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        const int r = ty * KB + i, c = tx * KB + j;
        sA[r * (K + 1) + c] = acc[i][j] + (r == c ? a.lambda : 0.f);
      }
    if (tid < K) sb[tid] = bacc;
    __syncthreads();
    // Blocked Cholesky A = L L^T in place (lower triangle), panels of 16 columns: the 16 x 16
    // diagonal block is factored by one warp, the rows below are solved one thread per row, and
    // the trailing matrix gets a rank-16 update with a (KB-1) x (KB-1) register tile per thread.
    // Three block-wide barriers per panel instead of three per column.
    constexpr int LD = K + 1;
    for (int j0 = 0; j0 < K; j0 += 16) {
      if (tid < 32) {
        for (int j = 0; j < 16; ++j) {
          const float d = sqrtf(fmaxf(sA[(j0 + j) * LD + j0 + j], 1e-30f));
          const float inv = 1.f / d;
          float lij = 0.f;
          const bool below = tid < 16 && tid > j;
          __syncwarp();
          if (below) {
            lij = sA[(j0 + tid) * LD + j0 + j] * inv;
            sA[(j0 + tid) * LD + j0 + j] = lij;
          }
          if (tid == j) sA[(j0 + j) * LD + j0 + j] = d;
          __syncwarp();
          if (below)
            for (int c = j + 1; c <= tid; ++c)
              sA[(j0 + tid) * LD + j0 + c] -= lij * sA[(j0 + c) * LD + j0 + j];
          __syncwarp();
        }
      }
      __syncthreads();
      const int j1 = j0 + 16;
      const int m = K - j1;             // rows below the panel
      if (tid < m) {                    // L21 = A21 L11^-T, one row per thread
        float* rowp = sA + (j1 + tid) * LD + j0;
        float x[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          float v = rowp[c];
#pragma unroll
          for (int q = 0; q < c; ++q) v = fmaf(-x[q], sA[(j0 + c) * LD + j0 + q], v);
          x[c] = v / sA[(j0 + c) * LD + j0 + c];
        }
#pragma unroll
        for (int c = 0; c < 16; ++c) rowp[c] = x[c];
      }
      __syncthreads();
      if (m > 0) {                      // A22 -= L21 L21^T (lower triangle only)
        const int mb = m >> 4;
        float t[KB - 1 > 0 ? KB - 1 : 1][KB - 1 > 0 ? KB - 1 : 1];
#pragma unroll
        for (int i = 0; i < KB - 1; ++i)
#pragma unroll
          for (int j = 0; j < KB - 1; ++j) t[i][j] = 0.f;
#pragma unroll 4
        for (int q = 0; q < 16; ++q) {
          float lr[KB - 1 > 0 ? KB - 1 : 1], lc[KB - 1 > 0 ? KB - 1 : 1];
#pragma unroll
          for (int i = 0; i < KB - 1; ++i) {
            lr[i] = i < mb ? sA[(j1 + ty + 16 * i) * LD + j0 + q] : 0.f;
            lc[i] = i < mb ? sA[(j1 + tx + 16 * i) * LD + j0 + q] : 0.f;
          }
#pragma unroll
          for (int i = 0; i < KB - 1; ++i)
#pragma unroll
            for (int j = 0; j < KB - 1; ++j) t[i][j] = fmaf(lr[i], lc[j], t[i][j]);
        }
#pragma unroll
        for (int i = 0; i < KB - 1; ++i)
#pragma unroll
          for (int j = 0; j < KB - 1; ++j) {
            const int r = j1 + ty + 16 * i, c = j1 + tx + 16 * j;
            if (i < mb && j < mb && c <= r) sA[r * LD + c] -= t[i][j];
          }
      }
      __syncthreads();
    }
    // forward: L y = b, panel by panel (a warp solves the 16 x 16 block with shuffles)
    for (int j0 = 0; j0 < K; j0 += 16) {
      if (tid < 32) {
        float bv = tid < 16 ? sb[j0 + tid] : 0.f;
        for (int c = 0; c < 16; ++c) {
          const float yc = __shfl_sync(0xffffffffu, bv, c) / sA[(j0 + c) * LD + j0 + c];
          if (tid == c) bv = yc;
          else if (tid < 16 && tid > c) bv = fmaf(-sA[(j0 + tid) * LD + j0 + c], yc, bv);
        }
        if (tid < 16) sb[j0 + tid] = bv;
      }
      __syncthreads();
      const int j1 = j0 + 16;
      if (tid < K - j1) {
        float v = sb[j1 + tid];
#pragma unroll
        for (int q = 0; q < 16; ++q) v = fmaf(-sA[(j1 + tid) * LD + j0 + q], sb[j0 + q], v);
        sb[j1 + tid] = v;
      }
      __syncthreads();
    }
    // backward: L^T w = y, last panel first
    for (int j0 = K - 16; j0 >= 0; j0 -= 16) {
      if (tid < 32) {
        float bv = tid < 16 ? sb[j0 + tid] : 0.f;
        for (int c = 15; c >= 0; --c) {
          const float wc = __shfl_sync(0xffffffffu, bv, c) / sA[(j0 + c) * LD + j0 + c];
          if (tid == c) bv = wc;
          else if (tid < c) bv = fmaf(-sA[(j0 + c) * LD + j0 + tid], wc, bv);
        }
        if (tid < 16) sb[j0 + tid] = bv;
      }
      __syncthreads();
      if (tid < j0) {
        float v = sb[tid];
#pragma unroll
        for (int q = 0; q < 16; ++q) v = fmaf(-sA[(j0 + q) * LD + tid], sb[j0 + q], v);
        sb[tid] = v;
      }
      __syncthreads();
    }
    if (tid < a.k) a.W[(long long)u * a.k + tid] = sb[tid];
    __syncthreads();
  }
}

template <int KB>
int launch(const AlsArgs& a, int blocks, cudaStream_t stream) {
  constexpr int K = 16 * KB;
  size_t smem = (size_t)(K * (K + 1) + K + 8 * K + 8) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(als_kernel<KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  als_kernel<KB><<<blocks, 256, smem, stream>>>(a);
  return pcl_last_error();
}

}  // namespace

// k <= 128.  Work items are segments (seg_user, [seg_begin, seg_end)); a user with more than
// one segment needs user_slot[u] >= 0 and zeroed `scratch` (slots x (K*K + K) floats, K = k
// rounded up to 32/64/96/128) and `slot_count`.
PCL_API int pcl_als_solve(const int* seg_user, const long long* seg_begin, const long long* seg_end,
                          const int* user_nseg, const int* user_slot, const int* item_idx,
                          const float* rating, const float* H, float* W, float* scratch,
                          unsigned int* slot_count, long long n_seg, int k, float lambda, int blocks,
                          cudaStream_t stream) {
  if (n_seg <= 0) return 0;
  if (k <= 0 || k > 128) return (int)cudaErrorInvalidValue;
  AlsArgs a{seg_user, seg_begin, seg_end, user_nseg, user_slot, item_idx, rating, H, W, scratch,
            slot_count, n_seg, k, lambda};
  if (blocks <= 0) blocks = 148 * 3;   // three CTAs per SM: the phases of one system are latency bound
  if (n_seg < blocks) blocks = (int)n_seg;
  if (k <= 32) return launch<2>(a, blocks, stream);
  if (k <= 64) return launch<4>(a, blocks, stream);
  if (k <= 96) return launch<6>(a, blocks, stream);
  return launch<8>(a, blocks, stream);
}
