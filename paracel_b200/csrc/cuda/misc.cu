// Smaller kernels of the algorithm suite.
//   kmeans_accumulate  per-cluster sums and counts after the assignment GEMM
//                      (alg/clustering/kmeans/kmeans.hpp:127-133)
//   topk_rows          running per-row top-k of a similarity tile with a lower bound and
//                      self-exclusion (alg/recommendation/similarity_dense/sim_dense.hpp:84-101)
//   gram               H^T H of a tall-skinny block (alg/recommendation/svd/svd.hpp:137-148)
//   allreduce_sum      sum of a small vector over all ranks through peer memory (the
//                      MPI_Allreduce of loss / RMSE / likelihood scalars, lr.cpp:331-334,
//                      mf.hpp:104-106), one launch, bounded wait
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) kmeans_accumulate_kernel(const float* X, const int* assign,
                                                                long long n, int d, float* sums,
                                                                float* counts) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < n; i += nwarps) {
    const int c = assign[i];
    const float* x = X + i * d;
    float* s = sums + (long long)c * d;
    for (int j = lane; j < d; j += 32) atomicAdd(s + j, x[j]);
    if (lane == 0) atomicAdd(counts + c, 1.f);
  }
}

// d a multiple of 4 and at most 512, X and sums 16-byte aligned: a lane owns up to four 16-byte
// pieces of a row and adds each with one vector reduction (a quarter of the requests the L2 atomic
// units see with scalar adds).  A warp takes four points per step: the four cluster ids, then all
// row pieces, then the reductions, so four rows are in flight per warp instead of one.
template <int PIECES>
__global__ void __launch_bounds__(256) kmeans_accumulate_vec_kernel(const float* X, const int* assign,
                                                                    long long n, int d, float* sums,
                                                                    float* counts) {
  constexpr int P = 4;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i0 = warp * P; i0 < n; i0 += nwarps * P) {
    int c[P];
#pragma unroll
    for (int k = 0; k < P; ++k) c[k] = (i0 + k < n) ? __ldg(assign + i0 + k) : -1;
    float4 x[P][PIECES];
#pragma unroll
    for (int k = 0; k < P; ++k)
#pragma unroll
      for (int q = 0; q < PIECES; ++q) {
        const int j = (q * 32 + lane) * 4;
        if (c[k] >= 0 && j < d) x[k][q] = __ldcs(reinterpret_cast<const float4*>(X + (i0 + k) * d + j));
      }
#pragma unroll
    for (int k = 0; k < P; ++k) {
      if (c[k] < 0) continue;
      float* s = sums + (long long)c[k] * d;
#pragma unroll
      for (int q = 0; q < PIECES; ++q) {
        const int j = (q * 32 + lane) * 4;
        if (j < d)
          asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(s + j), "f"(x[k][q].x),
                       "f"(x[k][q].y), "f"(x[k][q].z), "f"(x[k][q].w)
                       : "memory");
      }
      if (lane == 0) atomicAdd(counts + c[k], 1.f);
    }
  }
}

// Lane i of the warp holds the i-th best (value, id) of its row, best first.
__global__ void __launch_bounds__(256) topk_rows_kernel(const float* S, long long ldS, int m, int n,
                                                        const long long* row_ids,
                                                        const long long* col_ids, float lower, int k,
                                                        float* best_val, long long* best_idx) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int r = warp; r < m; r += nwarps) {
    float v = -3.402823466e38f;
    long long id = -1;
    if (lane < k) { v = best_val[(long long)r * k + lane]; id = best_idx[(long long)r * k + lane]; }
    const long long self = row_ids ? row_ids[r] : -1;
    const float* row = S + (long long)r * ldS;
    for (int c0 = 0; c0 < n; c0 += 32) {
      const int c = c0 + lane;
      float x = -3.402823466e38f;
      long long cid = -1;
      if (c < n) {
        x = row[c];
        cid = col_ids ? col_ids[c] : c;
      }
      const float kth = __shfl_sync(0xffffffffu, v, k - 1);
      unsigned cand = __ballot_sync(0xffffffffu, c < n && x >= lower && x > kth && cid != self);
      while (cand) {
        const int src = __ffs(cand) - 1;
        cand &= cand - 1;
        const float xv = __shfl_sync(0xffffffffu, x, src);
        const long long xi = __shfl_sync(0xffffffffu, cid, src);
        const float cur_kth = __shfl_sync(0xffffffffu, v, k - 1);
        if (!(xv > cur_kth)) continue;  // warp-uniform
        // position = number of entries that stay ahead of the newcomer
        const unsigned ahead = __ballot_sync(0xffffffffu, lane < k && v >= xv);
        const int pos = __popc(ahead);
        const float vup = __shfl_up_sync(0xffffffffu, v, 1);
        const long long iup = __shfl_up_sync(0xffffffffu, id, 1);
        if (lane > pos && lane < k) { v = vup; id = iup; }
        if (lane == pos) { v = xv; id = xi; }
      }
    }
    if (lane < k) { best_val[(long long)r * k + lane] = v; best_idx[(long long)r * k + lane] = id; }
  }
}

template <int KB>
__global__ void __launch_bounds__(256) gram_kernel(const float* H, long long n, int k, float* out) {
  constexpr int K = 16 * KB;
  __shared__ float sh[8 * K];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float acc[KB][KB];
#pragma unroll
  for (int i = 0; i < KB; ++i)
#pragma unroll
    for (int j = 0; j < KB; ++j) acc[i][j] = 0.f;
  for (long long r0 = (long long)blockIdx.x * 8; r0 < n; r0 += (long long)gridDim.x * 8) {
    const int cnt = (int)((n - r0) < 8 ? (n - r0) : 8);
    __syncthreads();
    for (int e = tid; e < cnt * K; e += 256) {
      const int r = e / K, c = e % K;
      sh[e] = (c < k) ? H[(r0 + r) * k + c] : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < cnt; ++r) {
#pragma unroll
      for (int i = 0; i < KB; ++i)
#pragma unroll
        for (int j = 0; j < KB; ++j)
          acc[i][j] = fmaf(sh[r * K + ty * KB + i], sh[r * K + tx * KB + j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < KB; ++i)
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const int r = ty * KB + i, c = tx * KB + j;
      if (r < k && c < k && acc[i][j] != 0.f) atomicAdd(out + (long long)r * k + c, acc[i][j]);
    }
}

struct ArArgs {
  const double* in;          // n values of this rank
  double* out;               // n sums
  int n;
  double* const* slots;      // world pointers: each rank's 2 x nmax staging area
  long long* const* flags;   // world pointers: each rank's flag array (world entries)
  const long long* my_flags; // this rank's flag array
  int world, rank, nmax;
  long long epoch;
  unsigned long long timeout_ns;
  PclStatus* status;
};

__global__ void __launch_bounds__(256) allreduce_sum_kernel(ArArgs a) {
  __shared__ int ok;
  const int par = (int)(a.epoch & 1);
  double* mine = a.slots[a.rank] + (long long)par * a.nmax;
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) mine[i] = a.in[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) pcl_st_release_sys(a.flags[threadIdx.x] + a.rank, a.epoch);
  if (threadIdx.x == 0)
    ok = pcl_wait_min_clock(a.my_flags, a.world, a.epoch, a.timeout_ns, a.status, a.rank, 30) ? 1 : 0;
  __syncthreads();
  if (!ok) return;
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
    double s = 0.0;
    for (int r = 0; r < a.world; ++r) {
      double v;
      asm volatile("ld.relaxed.sys.global.f64 %0, [%1];" : "=d"(v) : "l"(a.slots[r] + (long long)par * a.nmax + i));
      s += v;
    }
    a.out[i] = s;
  }
}

}  // namespace

PCL_API int pcl_kmeans_accumulate(const float* X, const int* assign, long long n, int d, float* sums,
                                  float* counts, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const bool vec = (d % 4 == 0) && d <= 512 && (((uintptr_t)X | (uintptr_t)sums) & 15) == 0;
  if (vec) {
    blocks = (n + 31) / 32;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (d <= 128) kmeans_accumulate_vec_kernel<1><<<(int)blocks, 256, 0, stream>>>(X, assign, n, d, sums, counts);
    else if (d <= 256) kmeans_accumulate_vec_kernel<2><<<(int)blocks, 256, 0, stream>>>(X, assign, n, d, sums, counts);
    else kmeans_accumulate_vec_kernel<4><<<(int)blocks, 256, 0, stream>>>(X, assign, n, d, sums, counts);
  } else {
    kmeans_accumulate_kernel<<<(int)blocks, 256, 0, stream>>>(X, assign, n, d, sums, counts);
  }
  return pcl_last_error();
}

// best_val (m x k, initialised to -FLT_MAX) / best_idx (m x k, -1) are updated with the columns
// of the tile S (m x n, leading dimension ldS); k <= 32.
PCL_API int pcl_topk_rows(const float* S, long long ldS, int m, int n, const long long* row_ids,
                          const long long* col_ids, float lower, int k, float* best_val,
                          long long* best_idx, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || k > 32) return (int)cudaErrorInvalidValue;
  int blocks = (m + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  topk_rows_kernel<<<blocks, 256, 0, stream>>>(S, ldS, m, n, row_ids, col_ids, lower, k, best_val, best_idx);
  return pcl_last_error();
}

// out (k x k, accumulated into; zero it first) += H^T H for H [n x k], k <= 128.
PCL_API int pcl_gram(const float* H, long long n, int k, float* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (k <= 0 || k > 128) return (int)cudaErrorInvalidValue;
  long long blocks = (n + 63) / 64;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (k <= 32) gram_kernel<2><<<(int)blocks, 256, 0, stream>>>(H, n, k, out);
  else if (k <= 64) gram_kernel<4><<<(int)blocks, 256, 0, stream>>>(H, n, k, out);
  else if (k <= 96) gram_kernel<6><<<(int)blocks, 256, 0, stream>>>(H, n, k, out);
  else gram_kernel<8><<<(int)blocks, 256, 0, stream>>>(H, n, k, out);
  return pcl_last_error();
}

PCL_API int pcl_allreduce_sum_f64(const double* in, double* out, int n, double* const* slots,
                                  long long* const* flags, const long long* my_flags, int world,
                                  int rank, int nmax, long long epoch, unsigned long long timeout_ns,
                                  PclStatus* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > nmax || world > 256) return (int)cudaErrorInvalidValue;
  ArArgs a{in, out, n, slots, flags, my_flags, world, rank, nmax, epoch, timeout_ns, status};
  allreduce_sum_kernel<<<1, 256, 0, stream>>>(a);
  return pcl_last_error();
}

// ---------------------------------------------------------------------------------------------
// Range check of an id array that a later kernel will use as an index without looking at it
// again (rating streams, CSR column arrays, word ids, topic assignments): run once when the
// data is loaded.  The first id outside [lo, hi) is recorded in the status block (code 2,
// wait_id 110, expected = position, seen = id); `skip` is a value that is allowed although it
// is out of range (padding markers), pass lo to allow none.
namespace {
template <typename T>
__global__ void validate_ids_kernel(const T* ids, long long n, long long lo, long long hi,
                                    long long skip, PclStatus* st, int rank) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long g = (long long)ids[i];
    if ((g < lo || g >= hi) && g != skip) pcl_report_bad_id(st, rank, 110, i, g);
  }
}
}  // namespace

PCL_API int pcl_validate_ids(const void* ids, int is64, long long n, long long lo, long long hi,
                             long long skip, PclStatus* status, int rank, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (status == nullptr) return (int)cudaErrorInvalidValue;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (is64)
    validate_ids_kernel<long long><<<(int)blocks, 256, 0, stream>>>(
        static_cast<const long long*>(ids), n, lo, hi, skip, status, rank);
  else
    validate_ids_kernel<int><<<(int)blocks, 256, 0, stream>>>(static_cast<const int*>(ids), n, lo,
                                                              hi, skip, status, rank);
  return pcl_last_error();
}
