// Sparse keyed pull / push of fixed-width rows against a table that is sharded
// over the HBM of all ranks (row g lives on rank g % world at local row
// g / world).  This is the device replacement of paracel_read_multi /
// paracel_bupdate_multi (reference: include/ps.hpp:482-534, 810-871 and the
// per-row loops of alg/recommendation/matrix_factorization/mf.hpp:202-262):
// the all-to-all "dispatch" is the address computation, the row gather is a
// 128-bit peer load over NVLink, and the "combine" is a vector reduction issued
// straight into the owner's shard, where the registered handler (add / scaled
// add / max) is applied by the L2 atomic unit of the owner GPU.
//
// The pull kernel can also carry the SSP staleness wait (bounded spin on the
// clock words that peers store into this GPU's memory), so that "wait until
// nobody is more than s clocks behind, then read" is one launch.
//
// Measured and not kept: four rows in flight per lane group in the pull and two in the push (ids of
// all rows, then all loads, then the stores / reductions) with 32-bit owner arithmetic.  On one
// GPU the pull went from 0.56 to 0.61 ms and the push from 0.70 to 0.84 ms for two million rows of
// 512 bytes: one row per group with 64 resident warps per SM already keeps the memory system busy.
#include "common.cuh"

namespace {

enum Handler { H_ADD = 0, H_SCALED_ADD = 1, H_MAX = 2, H_ASSIGN = 3 };

struct PullArgs {
  const long long* ids;      // n global row ids
  float* const* shards;      // world pointers (device array)
  int world;
  int D;                     // floats per row, multiple of 4
  long long n;
  float* dst;                // n x D working copy
  float* dst0;               // n x D snapshot (may be null)
  const long long* clocks;   // SSP clocks in local memory (may be null)
  long long target;          // wait for min(clocks) >= target (<=0: no wait)
  unsigned long long timeout_ns;
  PclStatus* status;
  int rank;
  long long rows;            // table extent: ids outside [0, rows) are reported and skipped
};

__global__ void __launch_bounds__(256) rows_pull_kernel(PullArgs a) {
  __shared__ int ok;
  if (a.clocks != nullptr && a.target > 0) {
    if (threadIdx.x == 0)
      ok = pcl_wait_min_clock(a.clocks, a.world, a.target, a.timeout_ns, a.status, a.rank, 1)
               ? 1 : 0;
    __syncthreads();
    if (!ok) return;
  }
  const int vec_per_row = a.D >> 2;
  // threads per row: largest power of two <= min(32, vec_per_row)
  int tpr = 32;
  while (tpr > vec_per_row) tpr >>= 1;
  const int rows_per_block = blockDim.x / tpr;
  const int sub = threadIdx.x % tpr;
  const int rib = threadIdx.x / tpr;
  for (long long row = (long long)blockIdx.x * rows_per_block + rib; row < a.n;
       row += (long long)gridDim.x * rows_per_block) {
    long long g = a.ids[row];
    if (g < 0 || g >= a.rows) {
      if (sub == 0) pcl_report_bad_id(a.status, a.rank, 101, row, g);
      continue;
    }
    int owner = (int)(g % a.world);
    long long lrow = g / a.world;
    const float* src = a.shards[owner] + lrow * a.D;
    float* d = a.dst + row * a.D;
    float* d0 = a.dst0 ? a.dst0 + row * a.D : nullptr;
    for (int v = sub; v < vec_per_row; v += tpr) {
      float4 x = pcl_ld_sys4(src + 4 * v);
      *reinterpret_cast<float4*>(d + 4 * v) = x;
      if (d0) *reinterpret_cast<float4*>(d0 + 4 * v) = x;
    }
  }
}

struct PushArgs {
  const long long* ids;
  float* const* shards;
  int world;
  int D;
  long long n;
  float* cur;          // n x D current working copy
  float* old;          // n x D snapshot taken at pull time; may be null (delta = cur)
  const float* wgt;    // n per-row weights or null (=1)
  float scale;         // extra scale for H_SCALED_ADD
  int handler;
  int refresh_old;     // write old = cur after pushing
  long long start;     // rows are visited in the order start, start+1, .., n-1, 0, .., start-1
  long long rows;      // table extent
  PclStatus* status;   // bad ids are reported here; a non-zero code on entry cancels the push
  int rank;
};

// Maximum handler on a row that may live in a peer GPU: system-scope integer atomics on the
// order-preserving bit pattern.  Precondition: neither value is NaN.  -0.0f is stored as +0.0f
// so that the signed / unsigned comparison orders the two zeros consistently.
__device__ __forceinline__ void atomic_max_f32(float* p, float v) {
  if (v == 0.f) v = 0.f;
  if (v >= 0.f) atomicMax_system(reinterpret_cast<int*>(p), __float_as_int(v));
  else atomicMin_system(reinterpret_cast<unsigned int*>(p), __float_as_uint(v));
}

__device__ __forceinline__ void st_sys4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(256) rows_push_kernel(PushArgs a) {
  // a wait of this round that timed out (or a bad id) left the working copies stale: push nothing
  if (pcl_status_code(a.status) != 0) return;
  const int vec_per_row = a.D >> 2;
  int tpr = 32;
  while (tpr > vec_per_row) tpr >>= 1;
  const int rows_per_block = blockDim.x / tpr;
  const int sub = threadIdx.x % tpr;
  const int rib = threadIdx.x / tpr;
  for (long long it = (long long)blockIdx.x * rows_per_block + rib; it < a.n;
       it += (long long)gridDim.x * rows_per_block) {
    // ranks that hold the same rows (same grid row / column of the loader's partition) pass
    // different `start` values, so that they do not reduce into the same destination rows at
    // the same moment
    long long row = it + a.start;
    if (row >= a.n) row -= a.n;
    long long g = a.ids[row];
    if (g < 0 || g >= a.rows) {
      if (sub == 0) pcl_report_bad_id(a.status, a.rank, 102, row, g);
      continue;
    }
    int owner = (int)(g % a.world);
    long long lrow = g / a.world;
    float* dstp = a.shards[owner] + lrow * a.D;
    float w = a.wgt ? a.wgt[row] : 1.f;
    if (a.handler == H_SCALED_ADD) w *= a.scale;
    float* c = a.cur + row * a.D;
    float* o = a.old ? a.old + row * a.D : nullptr;
    for (int v = sub; v < vec_per_row; v += tpr) {
      float4 x = *reinterpret_cast<const float4*>(c + 4 * v);
      float4 d = x;
      if (o) {
        float4 y = *reinterpret_cast<const float4*>(o + 4 * v);
        d.x -= y.x; d.y -= y.y; d.z -= y.z; d.w -= y.w;
      }
      if (a.handler == H_MAX) {
        atomic_max_f32(dstp + 4 * v + 0, x.x);
        atomic_max_f32(dstp + 4 * v + 1, x.y);
        atomic_max_f32(dstp + 4 * v + 2, x.z);
        atomic_max_f32(dstp + 4 * v + 3, x.w);
      } else if (a.handler == H_ASSIGN) {
        st_sys4(dstp + 4 * v, x);
      } else {
        d.x *= w; d.y *= w; d.z *= w; d.w *= w;
        if (d.x != 0.f || d.y != 0.f || d.z != 0.f || d.w != 0.f)
          pcl_red_add4_sys(dstp + 4 * v, d);
      }
    }
  }
  // Snapshot refresh (old = cur) as a second sweep over the same elements.  Interleaving these
  // stores with the system-scope reductions of the first sweep made the kernel about five times
  // slower on NVLink (1.5 ms instead of 0.2 ms for one million rows of 512 bytes).
  if (a.old != nullptr && a.refresh_old) {
    for (long long it = (long long)blockIdx.x * rows_per_block + rib; it < a.n;
         it += (long long)gridDim.x * rows_per_block) {
      long long row = it + a.start;
      if (row >= a.n) row -= a.n;
      const float* c = a.cur + row * a.D;
      float* o = a.old + row * a.D;
      for (int v = sub; v < vec_per_row; v += tpr)
        *reinterpret_cast<float4*>(o + 4 * v) = *reinterpret_cast<const float4*>(c + 4 * v);
    }
  }
}

// Scalar tables (biases, counts): one element per id.
struct ScalarArgs {
  const long long* ids;
  float* const* shards;
  int world;
  long long n;
  float* cur;
  float* old;
  const float* wgt;
  int refresh_old;
  int handler;
  long long rows;
  PclStatus* status;
  int rank;
};

__global__ void scalars_pull_kernel(ScalarArgs a) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    long long g = a.ids[i];
    if (g < 0 || g >= a.rows) {
      pcl_report_bad_id(a.status, a.rank, 103, i, g);
      continue;
    }
    const float* src = a.shards[(int)(g % a.world)] + g / a.world;
    float x;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(x) : "l"(src));
    a.cur[i] = x;
    if (a.old) a.old[i] = x;
  }
}

__global__ void scalars_push_kernel(ScalarArgs a) {
  if (pcl_status_code(a.status) != 0) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    long long g = a.ids[i];
    if (g < 0 || g >= a.rows) {
      pcl_report_bad_id(a.status, a.rank, 104, i, g);
      continue;
    }
    float* dstp = a.shards[(int)(g % a.world)] + g / a.world;
    float x = a.cur[i];
    if (a.handler == H_MAX) {
      atomic_max_f32(dstp, x);
      continue;
    }
    if (a.handler == H_ASSIGN) {
      asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dstp), "f"(x) : "memory");
      continue;
    }
    float d = a.old ? x - a.old[i] : x;
    if (a.wgt) d *= a.wgt[i];
    if (d != 0.f)
      asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(dstp), "f"(d) : "memory");
  }
  if (a.old != nullptr && a.refresh_old) {   // second sweep, see rows_push_kernel
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n;
         i += (long long)gridDim.x * blockDim.x)
      a.old[i] = a.cur[i];
  }
}

// int32 rows (LDA word-topic counts): pull = copy, push = integer add of deltas.
struct IRowArgs {
  const long long* ids;
  int* const* shards;
  int world;
  int D;  // ints per row, multiple of 4
  long long n;
  int* cur;
  int* old;
  int refresh_old;
  long long rows;
  PclStatus* status;
  int rank;
};

__global__ void __launch_bounds__(256) irows_pull_kernel(IRowArgs a) {
  const int vec_per_row = a.D >> 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long row = (long long)blockIdx.x * wpb + warp; row < a.n;
       row += (long long)gridDim.x * wpb) {
    long long g = a.ids[row];
    if (g < 0 || g >= a.rows) {
      if (lane == 0) pcl_report_bad_id(a.status, a.rank, 105, row, g);
      continue;
    }
    const int* src = a.shards[(int)(g % a.world)] + (g / a.world) * a.D;
    for (int v = lane; v < vec_per_row; v += 32) {
      int4 x;
      asm volatile("ld.relaxed.sys.global.v4.s32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
                   : "l"(src + 4 * v));
      *reinterpret_cast<int4*>(a.cur + row * a.D + 4 * v) = x;
      if (a.old) *reinterpret_cast<int4*>(a.old + row * a.D + 4 * v) = x;
    }
  }
}

__global__ void __launch_bounds__(256) irows_push_kernel(IRowArgs a) {
  if (pcl_status_code(a.status) != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long row = (long long)blockIdx.x * wpb + warp; row < a.n;
       row += (long long)gridDim.x * wpb) {
    long long g = a.ids[row];
    if (g < 0 || g >= a.rows) {
      if (lane == 0) pcl_report_bad_id(a.status, a.rank, 106, row, g);
      continue;
    }
    int* dstp = a.shards[(int)(g % a.world)] + (g / a.world) * a.D;
    for (int e = lane; e < a.D; e += 32) {
      int x = a.cur[row * a.D + e];
      int d = a.old ? x - a.old[row * a.D + e] : x;
      if (d != 0)
        asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(dstp + e), "r"(d)
                     : "memory");
    }
  }
  if (a.old != nullptr && a.refresh_old) {   // second sweep, see rows_push_kernel
    for (long long row = (long long)blockIdx.x * wpb + warp; row < a.n;
         row += (long long)gridDim.x * wpb)
      for (int e = lane; e < a.D; e += 32) a.old[row * a.D + e] = a.cur[row * a.D + e];
  }
}

inline int grid_for(long long work_items, int per_block, int max_blocks) {
  long long b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

}  // namespace

PCL_API int pcl_rows_pull_f32(const long long* ids, float* const* shards, int world, int D,
                              long long n, float* dst, float* dst0, const long long* clocks,
                              long long target, unsigned long long timeout_ns,
                              PclStatus* status, int rank, long long rows, cudaStream_t stream) {
  if (D <= 0 || (D & 3)) return (int)cudaErrorInvalidValue;
  if (n <= 0 && !(clocks && target > 0)) return 0;
  PullArgs a{ids, shards, world, D, n, dst, dst0, clocks, target, timeout_ns, status, rank, rows};
  int vec = D >> 2, tpr = 32;
  while (tpr > vec) tpr >>= 1;
  int grid = grid_for(n, 256 / tpr, 148 * 16);
  rows_pull_kernel<<<grid, 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_rows_push_f32(const long long* ids, float* const* shards, int world, int D,
                              long long n, float* cur, float* old, const float* wgt,
                              float scale, int handler, int refresh_old, long long start,
                              long long rows, PclStatus* status, int rank, cudaStream_t stream) {
  if (D <= 0 || (D & 3)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  if (start < 0 || start >= n) start = 0;
  PushArgs a{ids, shards, world, D, n, cur, old, wgt, scale, handler, refresh_old, start,
             rows, status, rank};
  int vec = D >> 2, tpr = 32;
  while (tpr > vec) tpr >>= 1;
  int grid = grid_for(n, 256 / tpr, 148 * 16);
  rows_push_kernel<<<grid, 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_scalars_pull_f32(const long long* ids, float* const* shards, int world,
                                 long long n, float* cur, float* old, long long rows,
                                 PclStatus* status, int rank, cudaStream_t stream) {
  if (n <= 0) return 0;
  ScalarArgs a{ids, shards, world, n, cur, old, nullptr, 0, H_ADD, rows, status, rank};
  scalars_pull_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_scalars_push_f32(const long long* ids, float* const* shards, int world,
                                 long long n, float* cur, float* old, const float* wgt,
                                 int refresh_old, int handler, long long rows, PclStatus* status,
                                 int rank, cudaStream_t stream) {
  if (n <= 0) return 0;
  ScalarArgs a{ids, shards, world, n, cur, old, wgt, refresh_old, handler, rows, status, rank};
  scalars_push_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_rows_pull_i32(const long long* ids, int* const* shards, int world, int D,
                              long long n, int* cur, int* old, long long rows, PclStatus* status,
                              int rank, cudaStream_t stream) {
  if (D <= 0 || (D & 3)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  IRowArgs a{ids, shards, world, D, n, cur, old, 0, rows, status, rank};
  irows_pull_kernel<<<grid_for(n, 8, 148 * 16), 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_rows_push_i32(const long long* ids, int* const* shards, int world, int D,
                              long long n, int* cur, int* old, int refresh_old, long long rows,
                              PclStatus* status, int rank, cudaStream_t stream) {
  if (D <= 0 || (D & 3)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  IRowArgs a{ids, shards, world, D, n, cur, old, refresh_old, rows, status, rank};
  irows_push_kernel<<<grid_for(n, 8, 148 * 16), 256, 0, stream>>>(a);
  return pcl_last_error();
}
