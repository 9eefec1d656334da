// Kernels of the device SVD (alternating least squares + Cholesky-QR; reference:
// alg/recommendation/svd/svd.hpp:137-181 for the products A.H and A^T.W that it forms with
// Eigen on every worker, 221-231 for the Cholesky-QR):
//
//   spmm_csr      out[r, :]  = sum_j A[r, c_j] * H[c_j, :]      (warp per row, K <= 128)
//   spmm_csr_t    out[c, :] += A[r, c] * W[r, :]                (vector reductions, fp32)
//   chol_factor   G = L L^T for a small K x K Gram matrix; writes R = L^T and T = L^-T so that
//                 Q = M T is orthonormal and M = Q R, and G^-1 = T T^T.  One CTA, fp64 in
//                 shared memory.  A pivot below the tolerance marks the matrix rank deficient in
//                 `info` (index of the pivot + 1) and the caller falls back to an
//                 eigen-decomposition.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) spmm_csr_kernel(const long long* __restrict__ row_ptr,
                                                       const int* __restrict__ cols,
                                                       const float* __restrict__ vals, long long n_rows,
                                                       const float* __restrict__ H, int K,
                                                       float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const bool on = 4 * lane < K;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < n_rows;
       r += (long long)gridDim.x * wpb) {
    const long long b = row_ptr[r], e = row_ptr[r + 1];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long p0 = b; p0 < e; p0 += 32) {
      // 32 entries of the row at a time: one coalesced load, then broadcasts
      const long long p = p0 + lane;
      const int c_l = p < e ? cols[p] : 0;
      const float v_l = p < e ? (vals ? vals[p] : 1.f) : 0.f;
      const int cnt = (int)((e - p0) < 32 ? (e - p0) : 32);
      for (int j = 0; j < cnt; ++j) {
        const int c = __shfl_sync(0xffffffffu, c_l, j);
        const float v = __shfl_sync(0xffffffffu, v_l, j);
        if (on) {
          const float4 h = *reinterpret_cast<const float4*>(H + (long long)c * K + 4 * lane);
          acc.x = fmaf(v, h.x, acc.x); acc.y = fmaf(v, h.y, acc.y);
          acc.z = fmaf(v, h.z, acc.z); acc.w = fmaf(v, h.w, acc.w);
        }
      }
    }
    if (on) *reinterpret_cast<float4*>(out + r * K + 4 * lane) = acc;
  }
}

__global__ void __launch_bounds__(256) spmm_csr_t_kernel(const long long* __restrict__ row_ptr,
                                                         const int* __restrict__ cols,
                                                         const float* __restrict__ vals, long long n_rows,
                                                         const float* __restrict__ W, int K,
                                                         float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const bool on = 4 * lane < K;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < n_rows;
       r += (long long)gridDim.x * wpb) {
    const long long b = row_ptr[r], e = row_ptr[r + 1];
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) w = *reinterpret_cast<const float4*>(W + r * K + 4 * lane);
    for (long long p0 = b; p0 < e; p0 += 32) {
      const long long p = p0 + lane;
      const int c_l = p < e ? cols[p] : 0;
      const float v_l = p < e ? (vals ? vals[p] : 1.f) : 0.f;
      const int cnt = (int)((e - p0) < 32 ? (e - p0) : 32);
      for (int j = 0; j < cnt; ++j) {
        const int c = __shfl_sync(0xffffffffu, c_l, j);
        const float v = __shfl_sync(0xffffffffu, v_l, j);
        if (on && v != 0.f)
          pcl_red_add4(out + (long long)c * K + 4 * lane, make_float4(v * w.x, v * w.y, v * w.z, v * w.w));
      }
    }
  }
}

// One CTA.  Shared memory: L (K x K doubles) and X = L^-1 (K x K doubles).
__global__ void __launch_bounds__(256) chol_factor_kernel(const float* __restrict__ G, int K,
                                                          float* __restrict__ T, float* __restrict__ R,
                                                          double rel_tol, int* __restrict__ info) {
  extern __shared__ double sd[];
  double* L = sd;
  double* X = sd + (size_t)K * K;
  __shared__ double s_diag, s_max;
  __shared__ int s_bad;
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int e = tid; e < K * K; e += nt) {
    const int i = e / K, j = e % K;
    L[e] = 0.5 * ((double)G[i * K + j] + (double)G[j * K + i]);   // symmetrise
    X[e] = 0.0;
  }
  if (tid == 0) { s_bad = 0; s_max = 0.0; }
  __syncthreads();
  if (tid == 0) {
    double m = 0.0;
    for (int i = 0; i < K; ++i) m = fmax(m, fabs(L[i * K + i]));
    s_max = m;
  }
  __syncthreads();
  // right-looking Cholesky on the lower triangle
  for (int j = 0; j < K; ++j) {
    if (tid == 0) {
      const double d = L[j * K + j];
      if (!(d > rel_tol * s_max) && s_bad == 0) s_bad = j + 1;
      s_diag = d > 0.0 ? sqrt(d) : 1.0;
    }
    __syncthreads();
    if (s_bad) break;
    const double dj = s_diag;
    for (int i = j + tid; i < K; i += nt) L[i * K + j] = (i == j) ? dj : L[i * K + j] / dj;
    __syncthreads();
    // trailing update: L[i][k] -= L[i][j] * L[k][j] for j < k <= i
    const int rem = K - j - 1;
    for (int e = tid; e < rem * rem; e += nt) {
      const int i = j + 1 + e / rem, k = j + 1 + e % rem;
      if (k <= i) L[i * K + k] -= L[i * K + j] * L[k * K + j];
    }
    __syncthreads();
  }
  if (s_bad) {
    if (tid == 0) *info = s_bad;
    return;
  }
  // X = L^-1 by forward substitution, one column per thread
  for (int c = tid; c < K; c += nt) {
    for (int i = c; i < K; ++i) {
      double s = (i == c) ? 1.0 : 0.0;
      for (int k = c; k < i; ++k) s -= L[i * K + k] * X[k * K + c];
      X[i * K + c] = s / L[i * K + i];
    }
  }
  __syncthreads();
  for (int e = tid; e < K * K; e += nt) {
    const int i = e / K, j = e % K;
    R[e] = (j >= i) ? (float)L[j * K + i] : 0.f;     // R = L^T (upper)
    T[e] = (j >= i) ? (float)X[j * K + i] : 0.f;     // T = (L^-1)^T (upper)
  }
  if (tid == 0) *info = 0;
}

}  // namespace

PCL_API int pcl_spmm_csr(const long long* row_ptr, const int* cols, const float* vals, long long n_rows,
                         const float* H, int K, float* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (K <= 0 || K > 128 || (K & 3)) return (int)cudaErrorInvalidValue;
  long long blocks = (n_rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  spmm_csr_kernel<<<(int)blocks, 256, 0, stream>>>(row_ptr, cols, vals, n_rows, H, K, out);
  return pcl_last_error();
}

PCL_API int pcl_spmm_csr_t(const long long* row_ptr, const int* cols, const float* vals, long long n_rows,
                           const float* W, int K, float* out, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (K <= 0 || K > 128 || (K & 3)) return (int)cudaErrorInvalidValue;
  long long blocks = (n_rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  spmm_csr_t_kernel<<<(int)blocks, 256, 0, stream>>>(row_ptr, cols, vals, n_rows, W, K, out);
  return pcl_last_error();
}

PCL_API int pcl_chol_factor(const float* G, int K, float* T, float* R, double rel_tol, int* info,
                            cudaStream_t stream) {
  if (K <= 0 || K > 112) return (int)cudaErrorInvalidValue;   // 2 K^2 doubles must fit in 227 KB
  const size_t smem = 2 * (size_t)K * K * sizeof(double);
  cudaError_t e = cudaFuncSetAttribute(chol_factor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  chol_factor_kernel<<<1, 256, smem, stream>>>(G, K, T, R, rel_tol, info);
  return pcl_last_error();
}
