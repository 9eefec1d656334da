// Gradient kernels of the linear models (logistic regression, ridge, sparse
// L1-regularised logistic regression / Lasso).
//
// Math (reference: alg/classification/logistic_regression/lr.cpp:69-72, 119-145;
// alg/regression/ridge/ridge.hpp:73-96; tool/lr_l1_serial.cpp:46-73 for the L1
// objective): residual r = y - h(theta.x) with h = sigmoid (logistic) or identity
// (ridge), gradient accumulator g = sum_rows r * x, loss = log-loss or squared error.
// The accumulated g is what the reference's "dgd" method pushes with one bupdate per
// round; here it is written straight into the delta vector that dense_bupdate reduces.
//
// Dense kernel: one warp per row, theta cached in shared memory, per-block partial
// gradient in shared memory, then a two-stage reduction through a scratch buffer
// (blocks x d partials, summed in block order by the last block) so that the result
// does not depend on atomics between blocks.
// Sparse kernel: CSR rows, one warp per row; features with index < hot_T (the most
// frequent ones after frequency renumbering) accumulate in shared memory per block,
// the others go to global memory with red.add.
#include <stdio.h>

#include "common.cuh"
#include <mutex>
#include "pcl_noalloc.h"

namespace {

struct DenseGradArgs {
  const float* X;      // n x d row-major
  const float* y;      // n
  const float* theta;  // d
  long long n;
  int d;
  int logistic;
  float* g;            // d, written (not accumulated)
  double* loss;        // 1, written
  float* scratch;      // gridDim.x * d partial gradients + gridDim.x loss partials (as 2 floats each)
  unsigned int* counter;  // zero before the first launch; the last block resets it
  int private_acc;     // 1: every warp owns a d-float accumulator in shared memory (no atomics)
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + __expf(-z)); }

// R > 0: d <= 32 * R, the row and this warp's gradient sums stay in registers (R values per lane,
// X is read exactly once); R == 0: any d, the row is read twice (the second time from cache).
template <int R>
__global__ void __launch_bounds__(256) dense_grad_kernel(DenseGradArgs a) {
  extern __shared__ float sm[];
  float* s_theta = sm;          // d
  float* s_g = sm + a.d;        // d
  __shared__ double s_loss[8];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int j = threadIdx.x; j < a.d; j += blockDim.x) s_theta[j] = a.theta[j];
  for (int j = threadIdx.x; j < (a.private_acc ? wpb : 1) * a.d; j += blockDim.x) s_g[j] = 0.f;
  __syncthreads();
  double loss = 0.0;
  float gacc[R > 0 ? R : 1];
#pragma unroll
  for (int t = 0; t < (R > 0 ? R : 1); ++t) gacc[t] = 0.f;
  for (long long row = (long long)blockIdx.x * wpb + warp; row < a.n; row += (long long)gridDim.x * wpb) {
    const float* x = a.X + row * a.d;
    float xr[R > 0 ? R : 1];
    float z = 0.f;
    if constexpr (R > 0) {
#pragma unroll
      for (int t = 0; t < R; ++t) {
        const int j = lane + 32 * t;
        xr[t] = j < a.d ? __ldg(x + j) : 0.f;
      }
#pragma unroll
      for (int t = 0; t < R; ++t) {
        const int j = lane + 32 * t;
        z = fmaf(xr[t], j < a.d ? s_theta[j] : 0.f, z);
      }
    } else {
      for (int j = lane; j < a.d; j += 32) z = fmaf(x[j], s_theta[j], z);
    }
    z = pcl_warp_sum(z);
    const float yy = a.y[row];
    float r;
    if (a.logistic) {
      const float h = sigmoidf_(z);
      r = yy - h;
      // log-loss with clamping so that a saturated sigmoid does not give inf
      const float hc = fminf(fmaxf(h, 1e-7f), 1.f - 1e-7f);
      loss += (yy == 1.f) ? -(double)__logf(hc) : -(double)__logf(1.f - hc);
    } else {
      r = yy - z;
      loss += (double)r * (double)r;
    }
    if constexpr (R > 0) {
#pragma unroll
      for (int t = 0; t < R; ++t) gacc[t] = fmaf(r, xr[t], gacc[t]);
    } else if (a.private_acc) {
      // entry j of this warp's accumulator is only ever touched by lane j % 32 of this warp
      float* gw = s_g + (long long)warp * a.d;
      for (int j = lane; j < a.d; j += 32) gw[j] = fmaf(r, x[j], gw[j]);
    } else {
      for (int j = lane; j < a.d; j += 32) atomicAdd(&s_g[j], r * x[j]);
    }
  }
  if constexpr (R > 0) {   // registers -> this warp's slot in shared memory
    float* gw = s_g + (long long)warp * a.d;
#pragma unroll
    for (int t = 0; t < R; ++t) {
      const int j = lane + 32 * t;
      if (j < a.d) gw[j] = gacc[t];
    }
  }
  if (lane == 0) s_loss[warp] = loss;  // identical in every lane of the warp
  __syncthreads();
  float* part = a.scratch + (long long)blockIdx.x * a.d;
  for (int j = threadIdx.x; j < a.d; j += blockDim.x) {
    float v = s_g[j];
    if (a.private_acc)
      for (int w = 1; w < wpb; ++w) v += s_g[(long long)w * a.d + j];
    part[j] = v;
  }
  if (threadIdx.x == 0) {
    double l = 0.0;
    for (int w = 0; w < wpb; ++w) l += s_loss[w];
    reinterpret_cast<double*>(a.scratch + (((long long)gridDim.x * a.d + 1) & ~1LL))[blockIdx.x] = l;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.counter, 1u);
    is_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int j = threadIdx.x; j < a.d; j += blockDim.x) {
    float s = 0.f;
    for (unsigned int b = 0; b < gridDim.x; ++b) s += __ldcg(a.scratch + (long long)b * a.d + j);
    a.g[j] = s;
  }
  if (threadIdx.x == 0) {
    const double* lp = reinterpret_cast<const double*>(a.scratch + (((long long)gridDim.x * a.d + 1) & ~1LL));
    double l = 0.0;
    for (unsigned int b = 0; b < gridDim.x; ++b) l += __ldcg(lp + b);
    *a.loss = l;
    *a.counter = 0u;
  }
}

struct SparseGradArgs {
  const long long* row_ptr;  // n + 1
  const int* cols;
  const float* vals;         // null: all ones
  const float* y;
  const float* theta;        // full local copy
  long long n;
  int logistic;
  int hot_T;                 // feature ids < hot_T accumulate in shared memory
  float* g;                  // accumulated into (caller zeroes it)
  double* loss;              // accumulated into
};

// Hot features (ids below hot_T) accumulate per CTA in shared memory as 32-bit fixed point
// (2^-14 units, native integer atomics: a floating-point shared-memory atomic add is a
// compare-and-swap loop that retries under contention, and the hottest features are hit by
// most warps of a CTA at once).  |residual * value| <= a few units and a CTA adds at most a
// few hundred thousand terms per feature, so 17 integer bits are ample.
constexpr float SG_FX = 16384.f, SG_FXI = 1.f / 16384.f;
#ifndef SG_ROWS_N
#define SG_ROWS_N 4
#endif
constexpr int SG_ROWS = SG_ROWS_N;

// residual of one row from its margin z; adds the row's loss
__device__ __forceinline__ float sg_residual(const SparseGradArgs& a, float z, float yy, double& loss) {
  if (a.logistic) {
    const float h = sigmoidf_(z);
    const float hc = fminf(fmaxf(h, 1e-7f), 1.f - 1e-7f);
    loss += (yy == 1.f) ? -(double)__logf(hc) : -(double)__logf(1.f - hc);
    return yy - h;
  }
  const float r = yy - z;
  loss += (double)r * (double)r;
  return r;
}

__device__ __forceinline__ void sg_scatter(const SparseGradArgs& a, int* s_hot, int c, float t, bool fx_ok) {
  if (c < a.hot_T && fx_ok && fabsf(t) < 64.f) atomicAdd(&s_hot[c], __float2int_rn(t * SG_FX));
  else atomicAdd(a.g + c, t);
}

// A warp takes SG_ROWS rows per step.  A row is a chain of dependent long-latency accesses (row
// pointers, column ids, gather of theta, then the atomics), and with one row per warp the SM had
// only as many chains in flight as resident warps (long scoreboard 17 stall cycles per issue).
// Rows of up to 64 non-zeros keep their ids and values in registers between the margin and the
// scatter; longer rows take the loop form.
// Measured on 50 M x 2^24 with 40 non-zeros per row: 1 / 2 / 4 / 8 rows per step give 2.04 / 3.16 /
// 3.36 / 2.06 G samples/s (eight rows cost too many registers).
__global__ void __launch_bounds__(256) sparse_grad_kernel(SparseGradArgs a) {
  extern __shared__ int s_hot[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int j = threadIdx.x; j < a.hot_T; j += blockDim.x) s_hot[j] = 0;
  __syncthreads();
  double loss = 0.0;
  // squared-loss residuals are unbounded: keep those in floating point
  const bool fx_ok = a.logistic != 0;
  const long long stride = (long long)gridDim.x * wpb;
  for (long long row0 = (long long)blockIdx.x * wpb + warp; row0 < a.n; row0 += SG_ROWS * stride) {
    long long rb[SG_ROWS], re[SG_ROWS];
    bool shortrows = true;
#pragma unroll
    for (int k = 0; k < SG_ROWS; ++k) {
      const long long row = row0 + k * stride;
      const bool has = row < a.n;
      rb[k] = has ? a.row_ptr[row] : 0;
      re[k] = has ? a.row_ptr[row + 1] : 0;
      shortrows &= (re[k] - rb[k] <= 64);
    }
    if (shortrows) {
      // ids and values of all rows, then all gathers, then the reductions
      int c[2 * SG_ROWS];
      float v[2 * SG_ROWS], t[2 * SG_ROWS];
#pragma unroll
      for (int q = 0; q < 2 * SG_ROWS; ++q) {
        const long long p = rb[q >> 1] + (q & 1) * 32 + lane;
        const bool in = p < re[q >> 1];
        c[q] = in ? __ldg(a.cols + p) : -1;
        v[q] = (in && a.vals) ? __ldg(a.vals + p) : 1.f;
      }
#pragma unroll
      for (int q = 0; q < 2 * SG_ROWS; ++q) t[q] = c[q] >= 0 ? __ldg(a.theta + c[q]) : 0.f;
      float z[SG_ROWS];
#pragma unroll
      for (int k = 0; k < SG_ROWS; ++k) z[k] = fmaf(v[2 * k], t[2 * k], v[2 * k + 1] * t[2 * k + 1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < SG_ROWS; ++k) z[k] += __shfl_xor_sync(0xffffffffu, z[k], o);
#pragma unroll
      for (int k = 0; k < SG_ROWS; ++k) {
        const long long row = row0 + k * stride;
        if (row >= a.n) break;
        const float r = sg_residual(a, z[k], a.y[row], loss);
        if (c[2 * k] >= 0) sg_scatter(a, s_hot, c[2 * k], r * v[2 * k], fx_ok);
        if (c[2 * k + 1] >= 0) sg_scatter(a, s_hot, c[2 * k + 1], r * v[2 * k + 1], fx_ok);
      }
      continue;
    }
    for (int k = 0; k < SG_ROWS; ++k) {
      const long long row = row0 + k * stride;
      if (row >= a.n) break;
      float zz = 0.f;
      for (long long q = rb[k] + lane; q < re[k]; q += 32) {
        const float vv = a.vals ? a.vals[q] : 1.f;
        zz = fmaf(vv, __ldg(a.theta + a.cols[q]), zz);
      }
      zz = pcl_warp_sum(zz);
      const float r = sg_residual(a, zz, a.y[row], loss);
      for (long long q = rb[k] + lane; q < re[k]; q += 32) {
        const float vv = a.vals ? a.vals[q] : 1.f;
        sg_scatter(a, s_hot, a.cols[q], r * vv, fx_ok);
      }
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < a.hot_T; j += blockDim.x) {
    const int v = s_hot[j];
    if (v != 0) atomicAdd(a.g + j, (float)v * SG_FXI);
  }
  if (lane == 0 && loss != 0.0) atomicAdd(a.loss, loss);
}

template <int R>
int launch_dense_grad_r(const DenseGradArgs& a, int blocks, size_t smem, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(dense_grad_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  dense_grad_kernel<R><<<blocks, 256, smem, stream>>>(a);
  return pcl_last_error();
}

// rows of up to 1024 floats are kept in registers (needs the per-warp shared-memory slots)
int launch_dense_grad(const DenseGradArgs& a, int blocks, size_t smem, cudaStream_t stream) {
  if (a.private_acc && a.d <= 128) return launch_dense_grad_r<4>(a, blocks, smem, stream);
  if (a.private_acc && a.d <= 256) return launch_dense_grad_r<8>(a, blocks, smem, stream);
  if (a.private_acc && a.d <= 512) return launch_dense_grad_r<16>(a, blocks, smem, stream);
  if (a.private_acc && a.d <= 1024) return launch_dense_grad_r<32>(a, blocks, smem, stream);
  return launch_dense_grad_r<0>(a, blocks, smem, stream);
}

}  // namespace

// Number of floats of scratch the dense gradient needs for `blocks` blocks and dimension d.
PCL_API long long pcl_lr_dense_scratch_floats(int blocks, int d) {
  return (long long)blocks * d + 2LL * blocks + 4;
}

// g[d] = sum_rows (y - h(theta.x)) x, *loss = summed loss.  `scratch` must hold
// pcl_lr_dense_scratch_floats(blocks, d) floats (8-byte aligned); `counter` is one
// zero-initialised unsigned int that the kernel leaves at zero.  d <= 12000.
PCL_API int pcl_lr_dense_grad(const float* X, const float* y, const float* theta, long long n, int d,
                              int logistic, float* g, double* loss, float* scratch,
                              unsigned int* counter, int blocks, cudaStream_t stream) {
  if (n <= 0 || d <= 0) return (int)cudaErrorInvalidValue;
  if (d > 12000) return (int)cudaErrorInvalidValue;
  if (blocks <= 0) blocks = 148 * 2;
  long long need = (n + 7) / 8;
  if (need < blocks) blocks = (int)need;
  // per-warp accumulators (8 warps) when they fit into shared memory, else one shared accumulator
  const int private_acc = (9 * (size_t)d * sizeof(float) <= 200 * 1024) ? 1 : 0;
  DenseGradArgs a{X, y, theta, n, d, logistic, g, loss, scratch, counter, private_acc};
  size_t smem = (private_acc ? 9 : 2) * (size_t)d * sizeof(float);
  return launch_dense_grad(a, blocks, smem, stream);
}

PCL_API int pcl_lr_sparse_grad(const long long* row_ptr, const int* cols, const float* vals,
                               const float* y, const float* theta, long long n, int logistic,
                               int hot_T, float* g, double* loss, int blocks, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hot_T < 0 || hot_T > 24 * 1024) return (int)cudaErrorInvalidValue;
  SparseGradArgs a{row_ptr, cols, vals, y, theta, n, logistic, hot_T, g, loss};
  size_t smem = (size_t)hot_T * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(sparse_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  if (blocks <= 0) {
    // as many blocks as are resident at once (the kernel is bound by gather / atomic latency,
    // so every resident warp counts; the shared-memory table of hot features sets the limit)
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sparse_grad_kernel, 256, smem);
    if (e != cudaSuccess) return (int)e;
    blocks = 148 * (per_sm > 0 ? per_sm : 4);
  }
  long long need = (n + 7) / 8;
  if (need < blocks) blocks = (int)need;
  sparse_grad_kernel<<<blocks, 256, smem, stream>>>(a);
  return pcl_last_error();
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the dense gradient (declared in pcl_noalloc.h).
//
// Some hosts of this library may not call cudaMalloc at all: a serving process
// that handed all of its HBM to one arena at start-up, a plug-in that runs
// inside somebody else's memory pool, or a latency-critical loop where the
// implicit device synchronisation of cudaMalloc/cudaFree is not acceptable.  For
// them the block partials and the block counter of dense_grad_kernel live in
// the two file-scope device arrays below instead of a caller-provided scratch
// tensor.  The price: every GPU that loads this library carries the
// PCL_NOALLOC_MAX_FLOATS * 4 bytes (4 MiB) until the process exits, and all
// calls on one device share the array, so two calls that overlap on the GPU
// (different streams) would overwrite each other's partials.
static __device__ __align__(256) float g_noalloc_scratch[PCL_NOALLOC_MAX_FLOATS];
static __device__ __align__(256) unsigned int g_noalloc_counter[64];

namespace {
struct NoAllocSlot {
  float* scratch = nullptr;
  unsigned int* counter = nullptr;
  bool ready = false;
};
NoAllocSlot g_noalloc_slots[64];        // filled under g_noalloc_mutex, one entry per device
std::mutex g_noalloc_mutex;
thread_local char g_noalloc_msg[256] = "";   // last message of the calling host thread

int noalloc_fail(cudaError_t e, const char* what) {
  snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "pcl_lr_dense_grad_noalloc: %s failed: %s", what,
           cudaGetErrorString(e));
  return (int)e;
}
}  // namespace

PCL_API const char* pcl_lr_dense_grad_noalloc_error() { return g_noalloc_msg; }

PCL_API int pcl_lr_dense_grad_noalloc(const float* X, const float* y, const float* theta, long long n,
                                      int d, int logistic, float* g, double* loss, int blocks,
                                      cudaStream_t stream) {
  g_noalloc_msg[0] = 0;
  if (n <= 0 || d <= 0 || d > 12000) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "pcl_lr_dense_grad_noalloc: need n > 0 and 0 < d <= 12000 (got n=%lld d=%d)", n, d);
    return (int)cudaErrorInvalidValue;
  }
  if (blocks <= 0) blocks = 148 * 2;
  long long need_blocks = (n + 7) / 8;
  if (need_blocks < blocks) blocks = (int)need_blocks;
  const long long need = (long long)blocks * d + 2LL * blocks + 4;
  if (need > (long long)PCL_NOALLOC_MAX_FLOATS) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg),
             "pcl_lr_dense_grad_noalloc: %d blocks x d=%d needs %lld floats of scratch, the built-in "
             "array holds %d; use fewer blocks or pcl_lr_dense_grad with your own scratch",
             blocks, d, need, (int)PCL_NOALLOC_MAX_FLOATS);
    return (int)cudaErrorInvalidValue;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) {
    snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "pcl_lr_dense_grad_noalloc: device index %d not supported", dev);
    return (int)cudaErrorInvalidDevice;
  }
  NoAllocSlot& slot = g_noalloc_slots[dev];
  std::lock_guard<std::mutex> guard(g_noalloc_mutex);   // set-up and launch of one call at a time
  if (!slot.ready) {
    // One-time set-up for this device (it is the current device): translate the symbols
    // into device addresses.  In host code the array names are only stand-ins.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) {
      snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
      return (int)e;
    }
    slot.scratch = (float*)p;
    e = cudaGetSymbolAddress(&p, g_noalloc_counter);
    if (e != cudaSuccess) {
      snprintf(g_noalloc_msg, sizeof(g_noalloc_msg), "cudaGetSymbolAddress(counter) failed: %s", cudaGetErrorString(e));
      return (int)e;
    }
    slot.counter = (unsigned int*)p;
    slot.ready = true;
  }
  // the counter must start at zero whatever an earlier (possibly aborted) call left behind;
  // the partials are fully overwritten by the kernel before they are read
  e = cudaMemsetAsync(slot.counter, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return noalloc_fail(e, "cudaMemsetAsync(counter)");
  const int private_acc = (9 * (size_t)d * sizeof(float) <= 200 * 1024) ? 1 : 0;   // as pcl_lr_dense_grad
  DenseGradArgs a{X, y, theta, n, d, logistic, g, loss, slot.scratch, slot.counter, private_acc};
  size_t smem = (private_acc ? 9 : 2) * (size_t)d * sizeof(float);
  const int rc = launch_dense_grad(a, blocks, smem, stream);
  if (rc != 0) return noalloc_fail((cudaError_t)rc, "kernel launch");
  return 0;
}
