// Matrix-factorisation SGD pass over one rank's ratings (biased MF:
// r^ = clip(mu + b_u + b_i + W_u.H_i, 1, 5); reference update rule in
// alg/recommendation/matrix_factorization/mf.hpp:266-280, estimate 84-92).
//
// Layout: ratings are sorted user-major (the reference traverses its bigraph
// user by user as well) and cut into chunks of 32; one warp owns a chunk.  A
// lane holds D/32 consecutive floats of the row, so one row is one coalesced
// 128-bit load per lane for D = 128.  The user row stays in registers while the
// chunk stays on the same user and is written back once per user per chunk with
// a vector reduction; the item row is read (L1-bypassing) and updated with a
// vector reduction per rating.  Reductions (never plain stores) mean no update
// is lost although thousands of warps run concurrently.
//
// Concurrency weights: the reference averages the deltas of the workers that
// hold the same row (wgt = 1/#workers, mf.hpp:217-262).  Inside one GPU the
// "workers" are the resident warps, so each row's delta is scaled by
// 1 / max(1, expected number of warps that update this row at the same time)
// (su for user rows, si for item rows, precomputed from the row counts).
#include "common.cuh"

namespace {

struct MfArgs {
  const int* ru;   // local user index per rating (user-major sorted)
  const int* ri;   // local item index per rating
  const float* rr; // rating
  long long nnz;
  float* W;        // nU x D working copy
  float* H;        // nI x D working copy
  float* bu;       // nU
  float* bi;       // nI
  const float* su; // nU concurrency weights
  const float* si; // nI concurrency weights
  float mu, alpha, beta;
  long long nchunks;
  long long stride;  // coprime with nchunks: spreads the chunks of one heavy user in time
  double* sse;       // optional: += sum of squared pre-update errors (running training loss)
};

template <int VEC>
struct Row {
  float v[VEC];
};

template <int VEC>
__device__ __forceinline__ Row<VEC> load_row_cg(const float* p) {
  Row<VEC> r;
  if constexpr (VEC == 1) {
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(r.v[0]) : "l"(p));
  } else if constexpr (VEC == 2) {
    asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];" : "=f"(r.v[0]), "=f"(r.v[1]) : "l"(p));
  } else {
#pragma unroll
    for (int j = 0; j < VEC; j += 4) {
      float4 x = pcl_ldcg4(p + j);
      r.v[j] = x.x; r.v[j + 1] = x.y; r.v[j + 2] = x.z; r.v[j + 3] = x.w;
    }
  }
  return r;
}

template <int VEC>
__device__ __forceinline__ void red_row(float* p, const Row<VEC>& d) {
  if constexpr (VEC == 1) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(d.v[0]) : "memory");
  } else if constexpr (VEC == 2) {
    asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" ::"l"(p), "f"(d.v[0]), "f"(d.v[1])
                 : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < VEC; j += 4)
      pcl_red_add4(p + j, make_float4(d.v[j], d.v[j + 1], d.v[j + 2], d.v[j + 3]));
  }
}

template <int VEC>
__global__ void __launch_bounds__(256, 4) mf_sgd_kernel(MfArgs a) {
  constexpr int D = VEC * 32;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const float ab = a.alpha * a.beta;
  float sse = 0.f;

  for (long long c = warp; c < a.nchunks; c += nwarps) {
    const long long ch = (c * a.stride) % a.nchunks;
    const long long base = ch * 32;
    const long long rem = a.nnz - base;
    const int n = rem < 32 ? (int)rem : 32;
    int my_u = -1, my_i = 0;
    float my_r = 0.f;
    if (lane < n) {
      my_u = __ldg(a.ru + base + lane);
      my_i = __ldg(a.ri + base + lane);
      my_r = __ldg(a.rr + base + lane);
    }
    int cur_u = -1;
    Row<VEC> w, w0;
    float bu = 0.f, bu0 = 0.f, s_u = 1.f;
#pragma unroll
    for (int k = 0; k < VEC; ++k) { w.v[k] = 0.f; w0.v[k] = 0.f; }

    // software prefetch of the first item row
    int i_nxt = __shfl_sync(0xffffffffu, my_i, 0);
    Row<VEC> h_nxt = load_row_cg<VEC>(a.H + (long long)i_nxt * D + lane * VEC);
    float bi_nxt = __ldcg(a.bi + i_nxt);
    float si_nxt = __ldg(a.si + i_nxt);

    for (int j = 0; j < n; ++j) {
      const int u = __shfl_sync(0xffffffffu, my_u, j);
      const int i = i_nxt;
      const float r = __shfl_sync(0xffffffffu, my_r, j);
      Row<VEC> h = h_nxt;
      const float bi = bi_nxt;
      const float s_i = si_nxt;
      if (j + 1 < n) {
        i_nxt = __shfl_sync(0xffffffffu, my_i, j + 1);
        h_nxt = load_row_cg<VEC>(a.H + (long long)i_nxt * D + lane * VEC);
        bi_nxt = __ldcg(a.bi + i_nxt);
        si_nxt = __ldg(a.si + i_nxt);
      }
      if (u < 0) continue;  // padding entry (warp-uniform)
      if (u != cur_u) {
        if (cur_u >= 0) {
          Row<VEC> d;
#pragma unroll
          for (int k = 0; k < VEC; ++k) d.v[k] = s_u * (w.v[k] - w0.v[k]);
          red_row<VEC>(a.W + (long long)cur_u * D + lane * VEC, d);
          if (lane == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
        }
        cur_u = u;
        w = load_row_cg<VEC>(a.W + (long long)u * D + lane * VEC);
        w0 = w;
        bu = __ldcg(a.bu + u);
        bu0 = bu;
        s_u = __ldg(a.su + u);
      }
      float dot = 0.f;
#pragma unroll
      for (int k = 0; k < VEC; ++k) dot = fmaf(w.v[k], h.v[k], dot);
      dot = pcl_warp_sum(dot);
      float pred = a.mu + bu + bi + dot;
      pred = fminf(5.f, fmaxf(1.f, pred));
      const float e = r - pred;
      sse = fmaf(e, e, sse);
      const float a2e = 2.f * a.alpha * e;
      Row<VEC> dh;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float wk = w.v[k], hk = h.v[k];
        dh.v[k] = s_i * (a2e * wk - ab * hk);
        w.v[k] = wk + (a2e * hk - ab * wk);
      }
      red_row<VEC>(a.H + (long long)i * D + lane * VEC, dh);
      bu += a2e - ab * bu;
      if (lane == 0) atomicAdd(a.bi + i, s_i * (a2e - ab * bi));
    }
    if (cur_u >= 0) {
      Row<VEC> d;
#pragma unroll
      for (int k = 0; k < VEC; ++k) d.v[k] = s_u * (w.v[k] - w0.v[k]);
      red_row<VEC>(a.W + (long long)cur_u * D + lane * VEC, d);
      if (lane == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
    }
  }
  if (a.sse != nullptr && lane == 0 && sse != 0.f) atomicAdd(a.sse, (double)sse);
}

struct RmseArgs {
  const int* ru;
  const int* ri;
  const float* rr;
  long long nnz;
  const float* W;
  const float* H;
  const float* bu;
  const float* bi;
  float mu;
  double* out;  // out[0] += sum of squared errors
  float* pred;  // optional per-rating prediction
};

template <int VEC>
__global__ void __launch_bounds__(256) mf_rmse_kernel(RmseArgs a) {
  constexpr int D = VEC * 32;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  double acc = 0.0;
  for (long long j = warp; j < a.nnz; j += nwarps) {
    const int u = __ldg(a.ru + j), i = __ldg(a.ri + j);
    float dot = 0.f;
    if (u >= 0 && i >= 0) {
      const float* wp = a.W + (long long)u * D + lane * VEC;
      const float* hp = a.H + (long long)i * D + lane * VEC;
#pragma unroll
      for (int k = 0; k < VEC; ++k) dot = fmaf(wp[k], hp[k], dot);
    }
    dot = pcl_warp_sum(dot);
    float pred = a.mu;
    if (u >= 0 && i >= 0) {
      pred = a.mu + a.bu[u] + a.bi[i] + dot;
      pred = fminf(5.f, fmaxf(1.f, pred));
    }
    if (a.pred && lane == 0) a.pred[j] = pred;
    if (a.rr) {
      const float e = __ldg(a.rr + j) - pred;
      acc += (double)e * (double)e;
    }
  }
  if (a.out) {
    __shared__ double sm[8];
    if (lane == 0) sm[threadIdx.x >> 5] = acc;  // every lane holds the same acc
    __syncthreads();
    if (threadIdx.x == 0) {
      double s = 0.0;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) s += sm[k];
      atomicAdd(a.out, s);
    }
  }
}

}  // namespace

// One SGD pass over `nnz` user-major sorted ratings (entries with a negative
// user index are padding and are skipped; `sse`, if given, accumulates the
// squared pre-update errors).  D must be 32, 64, 128 or
// 256 (pad the factors with zeros otherwise: zero columns stay zero under the
// update rule).  `blocks` <= 0 selects 148 SMs x 4 resident blocks.
PCL_API int pcl_mf_sgd_pass(const int* ru, const int* ri, const float* rr, long long nnz,
                            float* W, float* H, float* bu, float* bi, const float* su,
                            const float* si, int D, float mu, float alpha, float beta,
                            long long stride, int blocks, double* sse, cudaStream_t stream) {
  if (nnz <= 0) return 0;
  MfArgs a;
  a.ru = ru; a.ri = ri; a.rr = rr; a.nnz = nnz;
  a.W = W; a.H = H; a.bu = bu; a.bi = bi; a.su = su; a.si = si;
  a.mu = mu; a.alpha = alpha; a.beta = beta;
  a.nchunks = (nnz + 31) / 32;
  a.stride = (stride > 0 && stride < a.nchunks) ? stride : 1;
  a.sse = sse;
  if (blocks <= 0) blocks = 148 * 4;
  long long need = (a.nchunks + 7) / 8;
  if (need < blocks) blocks = (int)need;
  switch (D) {
    case 32: mf_sgd_kernel<1><<<blocks, 256, 0, stream>>>(a); break;
    case 64: mf_sgd_kernel<2><<<blocks, 256, 0, stream>>>(a); break;
    case 128: mf_sgd_kernel<4><<<blocks, 256, 0, stream>>>(a); break;
    case 256: mf_sgd_kernel<8><<<blocks, 256, 0, stream>>>(a); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return pcl_last_error();
}

// Sum of squared errors of the clipped estimate over `nnz` ratings, added to
// out[0] (double, device).  Ratings whose user or item index is negative are
// predicted as mu (the reference does the same for unseen ids, mf.hpp:364-366).
// `rr` may be null (prediction only) and `pred` may be null.
PCL_API int pcl_mf_sse(const int* ru, const int* ri, const float* rr, long long nnz,
                       const float* W, const float* H, const float* bu, const float* bi,
                       int D, float mu, double* out, float* pred, cudaStream_t stream) {
  if (nnz <= 0) return 0;
  RmseArgs a{ru, ri, rr, nnz, W, H, bu, bi, mu, out, pred};
  long long need = (nnz + 7) / 8;
  int blocks = need < 148 * 8 ? (int)need : 148 * 8;
  switch (D) {
    case 32: mf_rmse_kernel<1><<<blocks, 256, 0, stream>>>(a); break;
    case 64: mf_rmse_kernel<2><<<blocks, 256, 0, stream>>>(a); break;
    case 128: mf_rmse_kernel<4><<<blocks, 256, 0, stream>>>(a); break;
    case 256: mf_rmse_kernel<8><<<blocks, 256, 0, stream>>>(a); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return pcl_last_error();
}
