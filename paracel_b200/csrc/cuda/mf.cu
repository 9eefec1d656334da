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
  int hot_T;         // local item indices < hot_T are replicated in shared memory
  int cpw;           // chunks per warp between two flushes of the hot replicas
  float flush_scale; // mixing weight of one CTA's hot-row delta (1 / #CTAs)
  // compact rating stream (optional, replaces ru / ri / rr): 4 bytes per rating + 12 per chunk
  const unsigned int* packed;  // item index (low 24 bits) | rating code (high 8 bits)
  const int* chdr;             // per chunk: first user index, increment mask, number of valid entries
  const float* rtable;         // rating value of each code
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

// Shared-memory replicas of the hottest item rows.  Local item indices are
// ordered so that the T most frequent items of the rank come first; a CTA keeps
// the current value `hv` and the value at the start of the period `hbase` of
// each of them (layout [row][k][lane], bank-conflict free for a warp).  Every
// `cpw` chunks per warp the CTA reduces flush_scale * (hv - hbase) into the
// global row, reloads it, and goes on: the hot rows see shared-memory atomics
// (parallel over all SMs) instead of thousands of same-address L2 atomics, at
// the price of a bounded staleness between CTAs -- the same parameter-mixing
// rule the reference applies between workers (mf.hpp:217-262).
template <int VEC>
__global__ void __launch_bounds__(512, 2) mf_sgd_kernel(MfArgs a) {
  constexpr int D = VEC * 32;
  extern __shared__ float smem[];
  const int T = a.hot_T;
  // value at the start of the mixing period (float) + fixed-point delta of the period (2^-22
  // units, integer shared-memory atomics: native, no retry loop under contention)
  int* hd = reinterpret_cast<int*>(smem);                     // T x D
  float* hbase = smem + (size_t)T * D;                        // T x D
  int* hbd = reinterpret_cast<int*>(hbase + (size_t)T * D);   // T
  float* hbb = reinterpret_cast<float*>(hbd + T);             // T
  constexpr float FX = 4194304.f, FXI = 1.f / 4194304.f;
  const int lane = threadIdx.x & 31;
  const int wic = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const float ab = a.alpha * a.beta;
  float sse = 0.f;

  const long long step = (long long)gridDim.x * wpc;
  // uniform iteration count for every warp of this CTA (barriers inside the loop)
  const long long cta_chunks = a.nchunks > blockIdx.x
      ? (a.nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const long long iters = (cta_chunks + wpc - 1) / wpc;

  for (long long it = 0; it < iters; ++it) {
    if (T > 0 && (it % a.cpw) == 0) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
        const int row = idx / D, e = idx % D;          // e = global element in the row
        const int sidx = row * D + (e % VEC) * 32 + (e / VEC);
        float* gp = a.H + (size_t)row * D + e;
        if (it > 0) {
          const int d = hd[sidx];
          if (d != 0) atomicAdd(gp, (float)d * (FXI * a.flush_scale));
        }
        hd[sidx] = 0;
        hbase[sidx] = __ldcg(gp);
      }
      for (int row = threadIdx.x; row < T; row += blockDim.x) {
        if (it > 0) {
          const int d = hbd[row];
          if (d != 0) atomicAdd(a.bi + row, (float)d * (FXI * a.flush_scale));
        }
        hbd[row] = 0;
        hbb[row] = __ldcg(a.bi + row);
      }
      __syncthreads();
    }
    const long long c = (long long)blockIdx.x + ((long long)wic + it * wpc) * gridDim.x;
    if (c >= a.nchunks) continue;  // warp-uniform; barriers above are still reached
    const long long base = c * 32;
    int my_u, my_i;
    float my_r;
    if (a.packed != nullptr) {
      // users of a user-major sorted chunk grow by 0 or 1 per rating: a base and a bit mask
      const unsigned int pk = __ldg(a.packed + base + lane);
      const int u_base = __ldg(a.chdr + 3 * c);
      const unsigned int inc = (unsigned int)__ldg(a.chdr + 3 * c + 1);
      const int n_valid = __ldg(a.chdr + 3 * c + 2);
      my_i = (int)(pk & 0xffffffu);
      my_r = __ldg(a.rtable + (pk >> 24));
      my_u = lane < n_valid ? u_base + __popc(inc & (0xffffffffu >> (31 - lane))) : -1;
    } else {
      my_u = __ldg(a.ru + base + lane);
      my_i = __ldg(a.ri + base + lane);
      my_r = __ldg(a.rr + base + lane);
    }
    int cur_u = -1;
    Row<VEC> w, w0;
    float bu = 0.f, bu0 = 0.f, s_u = 1.f;
#pragma unroll
    for (int k = 0; k < VEC; ++k) { w.v[k] = 0.f; w0.v[k] = 0.f; }

    // software prefetch of the first item row (cold rows only)
    int i_nxt = __shfl_sync(0xffffffffu, my_i, 0);
    float si_nxt = __ldg(a.si + i_nxt);
    Row<VEC> h_nxt;
    float bi_nxt = 0.f;
#pragma unroll
    for (int k = 0; k < VEC; ++k) h_nxt.v[k] = 0.f;
    if (i_nxt >= T) {
      h_nxt = load_row_cg<VEC>(a.H + (long long)i_nxt * D + lane * VEC);
      bi_nxt = __ldcg(a.bi + i_nxt);
    }

#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
      const int u = __shfl_sync(0xffffffffu, my_u, j);
      const int i = i_nxt;
      const float r = __shfl_sync(0xffffffffu, my_r, j);
      const bool hot = i < T;
      Row<VEC> h = h_nxt;
      float bi = bi_nxt;
      const float s_i = si_nxt;
      if (j + 1 < 32) {
        i_nxt = __shfl_sync(0xffffffffu, my_i, j + 1);
        si_nxt = __ldg(a.si + i_nxt);
        if (i_nxt >= T) {
          h_nxt = load_row_cg<VEC>(a.H + (long long)i_nxt * D + lane * VEC);
          bi_nxt = __ldcg(a.bi + i_nxt);
        }
      }
      if (u < 0) continue;  // padding entry (warp-uniform)
      if (hot) {
#pragma unroll
        for (int k = 0; k < VEC; ++k)
          h.v[k] = fmaf((float)hd[i * D + k * 32 + lane], FXI, hbase[i * D + k * 32 + lane]);
        bi = fmaf((float)hbd[i], FXI, hbb[i]);
      }
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
      const float dbi = s_i * (a2e - ab * bi);
      bu += a2e - ab * bu;
      if (hot) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) atomicAdd(&hd[i * D + k * 32 + lane], __float2int_rn(dh.v[k] * FX));
        if (lane == 0) atomicAdd(&hbd[i], __float2int_rn(dbi * FX));
      } else {
        red_row<VEC>(a.H + (long long)i * D + lane * VEC, dh);
        if (lane == 0) atomicAdd(a.bi + i, dbi);
        if (j + 1 < 32 && i_nxt == i) {  // the prefetched copy predates this update
#pragma unroll
          for (int k = 0; k < VEC; ++k) h_nxt.v[k] += dh.v[k];
          bi_nxt += dbi;
        }
      }
    }
    if (cur_u >= 0) {
      Row<VEC> d;
#pragma unroll
      for (int k = 0; k < VEC; ++k) d.v[k] = s_u * (w.v[k] - w0.v[k]);
      red_row<VEC>(a.W + (long long)cur_u * D + lane * VEC, d);
      if (lane == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
    }
  }
  if (T > 0) {  // final flush of the hot replicas
    __syncthreads();
    for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
      const int row = idx / D, e = idx % D;
      const int sidx = row * D + (e % VEC) * 32 + (e / VEC);
      const int d = hd[sidx];
      if (d != 0) atomicAdd(a.H + (size_t)row * D + e, (float)d * (FXI * a.flush_scale));
    }
    for (int row = threadIdx.x; row < T; row += blockDim.x) {
      const int d = hbd[row];
      if (d != 0) atomicAdd(a.bi + row, (float)d * (FXI * a.flush_scale));
    }
  }
  if (a.sse != nullptr && lane == 0 && sse != 0.f) atomicAdd(a.sse, (double)sse);
}

// Rank-128 variant with 8 lanes per rating: a warp works on four chunks at once, one per
// group of 8 lanes, and every lane keeps 16 floats of each 128-float row (elements
// c*32 + l*4 + t, c < 4, t < 4, i.e. four 128-bit loads per row).  A warp-wide instruction thus
// advances four ratings, which cuts the instructions per rating to about a quarter of the
// 32-lanes-per-rating form; the rest of the algorithm (register-resident user row, vector
// reductions for cold item rows, shared-memory replicas of the hot item rows with periodic
// mixing) is unchanged.  Hot rows are stored with a stride of 132 floats and the four groups
// visit the four floats of a 16-byte element in rotated order, so that the 32 lanes of one
// shared-memory atomic hit 32 different banks.
constexpr int G8_STRIDE = 132;

__global__ void __launch_bounds__(512, 1) mf_sgd_kernel_g8(MfArgs a) {
  constexpr int D = 128;
  extern __shared__ float smem[];
  const int T = a.hot_T;
  float* hv = smem;                               // T x 132
  float* hbase = hv + (size_t)T * G8_STRIDE;      // T x 132
  float* hb = hbase + (size_t)T * G8_STRIDE;      // T
  float* hbb = hb + T;                            // T
  const int lane = threadIdx.x & 31;
  const int g = lane >> 3;                        // group within the warp
  const int l = lane & 7;                         // lane within the group
  const unsigned gmask = 0xffu << (8 * g);
  const int gic = (threadIdx.x >> 5) * 4 + g;     // group index within the CTA
  const int gpc = (blockDim.x >> 5) * 4;          // groups per CTA
  const float ab = a.alpha * a.beta;
  float sse = 0.f;

  const long long cta_chunks = a.nchunks > blockIdx.x
      ? (a.nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const long long iters = (cta_chunks + gpc - 1) / gpc;

  for (long long it = 0; it < iters; ++it) {
    if (T > 0 && (it % a.cpw) == 0) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
        const int row = idx >> 7, e = idx & 127;
        const int sidx = row * G8_STRIDE + e;
        float* gp = a.H + (size_t)row * D + e;
        if (it > 0) {
          const float d = hv[sidx] - hbase[sidx];
          if (d != 0.f) atomicAdd(gp, d * a.flush_scale);
        }
        const float v = __ldcg(gp);
        hv[sidx] = v;
        hbase[sidx] = v;
      }
      for (int row = threadIdx.x; row < T; row += blockDim.x) {
        if (it > 0) {
          const float d = hb[row] - hbb[row];
          if (d != 0.f) atomicAdd(a.bi + row, d * a.flush_scale);
        }
        const float v = __ldcg(a.bi + row);
        hb[row] = v;
        hbb[row] = v;
      }
      __syncthreads();
    }
    const long long c = (long long)blockIdx.x + ((long long)gic + it * gpc) * gridDim.x;
    const bool active = c < a.nchunks;          // uniform within the group
    const long long base = active ? c * 32 : 0;
    int cur_u = -1;
    float w[16], w0[16];
    float bu = 0.f, bu0 = 0.f, s_u = 1.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) { w[k] = 0.f; w0[k] = 0.f; }

    int i_nxt = active ? __ldg(a.ri + base) : 0;
    float si_nxt = active ? __ldg(a.si + i_nxt) : 0.f;
    float h_nxt[16];
    float bi_nxt = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) h_nxt[k] = 0.f;
    if (active && i_nxt >= T) {
      const float* hp = a.H + (long long)i_nxt * D + l * 4;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const float4 x = pcl_ldcg4(hp + cc * 32);
        h_nxt[4 * cc] = x.x; h_nxt[4 * cc + 1] = x.y; h_nxt[4 * cc + 2] = x.z; h_nxt[4 * cc + 3] = x.w;
      }
      bi_nxt = __ldcg(a.bi + i_nxt);
    }

#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
      if (!active) break;
      const int u = __ldg(a.ru + base + j);
      const float r = __ldg(a.rr + base + j);
      const int i = i_nxt;
      const bool hot = i < T;
      float h[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) h[k] = h_nxt[k];
      float bi = bi_nxt;
      const float s_i = si_nxt;
      if (j + 1 < 32) {
        i_nxt = __ldg(a.ri + base + j + 1);
        si_nxt = __ldg(a.si + i_nxt);
        if (i_nxt >= T) {
          const float* hp = a.H + (long long)i_nxt * D + l * 4;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const float4 x = pcl_ldcg4(hp + cc * 32);
            h_nxt[4 * cc] = x.x; h_nxt[4 * cc + 1] = x.y; h_nxt[4 * cc + 2] = x.z; h_nxt[4 * cc + 3] = x.w;
          }
          bi_nxt = __ldcg(a.bi + i_nxt);
        }
      }
      if (u < 0) continue;  // padding entry (uniform within the group)
      if (hot) {
        const float* sp = hv + i * G8_STRIDE + l * 4;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float4 x = *reinterpret_cast<const float4*>(sp + cc * 32);
          h[4 * cc] = x.x; h[4 * cc + 1] = x.y; h[4 * cc + 2] = x.z; h[4 * cc + 3] = x.w;
        }
        bi = hb[i];
      }
      if (u != cur_u) {
        if (cur_u >= 0) {
          float* wp = a.W + (long long)cur_u * D + l * 4;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
            pcl_red_add4(wp + cc * 32, make_float4(s_u * (w[4 * cc] - w0[4 * cc]),
                                                   s_u * (w[4 * cc + 1] - w0[4 * cc + 1]),
                                                   s_u * (w[4 * cc + 2] - w0[4 * cc + 2]),
                                                   s_u * (w[4 * cc + 3] - w0[4 * cc + 3])));
          if (l == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
        }
        cur_u = u;
        const float* wp = a.W + (long long)u * D + l * 4;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const float4 x = pcl_ldcg4(wp + cc * 32);
          w[4 * cc] = x.x; w[4 * cc + 1] = x.y; w[4 * cc + 2] = x.z; w[4 * cc + 3] = x.w;
        }
#pragma unroll
        for (int k = 0; k < 16; ++k) w0[k] = w[k];
        bu = __ldcg(a.bu + u);
        bu0 = bu;
        s_u = __ldg(a.su + u);
      }
      float dot = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) dot = fmaf(w[k], h[k], dot);
      dot += __shfl_xor_sync(gmask, dot, 4);
      dot += __shfl_xor_sync(gmask, dot, 2);
      dot += __shfl_xor_sync(gmask, dot, 1);
      float pred = a.mu + bu + bi + dot;
      pred = fminf(5.f, fmaxf(1.f, pred));
      const float e = r - pred;
      sse = fmaf(e, e, sse);
      const float a2e = 2.f * a.alpha * e;
      float dh[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float wk = w[k], hk = h[k];
        dh[k] = s_i * (a2e * wk - ab * hk);
        w[k] = wk + (a2e * hk - ab * wk);
      }
      const float dbi = s_i * (a2e - ab * bi);
      bu += a2e - ab * bu;
      if (hot) {
        float* sp = hv + i * G8_STRIDE + l * 4;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const int t = (tt + g) & 3;   // rotated per group: 32 lanes -> 32 banks
            // dh index must be a compile-time constant per unrolled iteration: select by t
            const float v = (t == 0) ? dh[4 * cc] : (t == 1) ? dh[4 * cc + 1]
                          : (t == 2) ? dh[4 * cc + 2] : dh[4 * cc + 3];
            atomicAdd(sp + cc * 32 + t, v);
          }
        }
        if (l == 0) atomicAdd(&hb[i], dbi);
      } else {
        float* hp = a.H + (long long)i * D + l * 4;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
          pcl_red_add4(hp + cc * 32, make_float4(dh[4 * cc], dh[4 * cc + 1], dh[4 * cc + 2], dh[4 * cc + 3]));
        if (l == 0) atomicAdd(a.bi + i, dbi);
        if (j + 1 < 32 && i_nxt == i) {  // the prefetched copy predates this update
#pragma unroll
          for (int k = 0; k < 16; ++k) h_nxt[k] += dh[k];
          bi_nxt += dbi;
        }
      }
    }
    if (cur_u >= 0) {
      float* wp = a.W + (long long)cur_u * D + l * 4;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
        pcl_red_add4(wp + cc * 32, make_float4(s_u * (w[4 * cc] - w0[4 * cc]),
                                               s_u * (w[4 * cc + 1] - w0[4 * cc + 1]),
                                               s_u * (w[4 * cc + 2] - w0[4 * cc + 2]),
                                               s_u * (w[4 * cc + 3] - w0[4 * cc + 3])));
      if (l == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
    }
  }
  if (T > 0) {  // final flush of the hot replicas
    __syncthreads();
    for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
      const int row = idx >> 7, e = idx & 127;
      const int sidx = row * G8_STRIDE + e;
      const float d = hv[sidx] - hbase[sidx];
      if (d != 0.f) atomicAdd(a.H + (size_t)row * D + e, d * a.flush_scale);
    }
    for (int row = threadIdx.x; row < T; row += blockDim.x) {
      const float d = hb[row] - hbb[row];
      if (d != 0.f) atomicAdd(a.bi + row, d * a.flush_scale);
    }
  }
  // every lane of a group saw the same errors: one lane per group reports
  if (a.sse != nullptr && l == 0 && sse != 0.f) atomicAdd(a.sse, (double)sse);
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

// One SGD pass over `nnz` user-major sorted ratings, nnz a multiple of 32
// (entries with a negative user index are padding and are skipped; `sse`, if
// given, accumulates the squared pre-update errors).  D must be 32, 64, 128 or
// 256 (pad the factors with zeros otherwise: zero columns stay zero under the
// update rule).  `blocks` <= 0 selects 2 CTAs of 512 threads per SM.  Local
// item indices below `hot_T` are served from shared-memory replicas that are
// mixed into the global rows every `cpw` chunks per warp with weight
// `flush_scale` (<= 0: 1 / blocks).  `variant` 2 (D = 128 only) selects the experimental
// 8-lanes-per-rating kernel (one CTA per SM, up to 211 hot rows); measured slower than the
// default because its four groups per warp diverge on the hot / cold / user-switch branches.
// Compact stream: when `packed` is given, ru / ri / rr are ignored; rating j of chunk c has item
// packed[32c+j] & 0xffffff, value rtable[packed >> 24] and user chdr[3c] + popcount of the low
// j+1 bits of chdr[3c+1] (bit 0 is always clear); entries j >= chdr[3c+2] are padding.
PCL_API int pcl_mf_sgd_pass(const int* ru, const int* ri, const float* rr, long long nnz,
                            float* W, float* H, float* bu, float* bi, const float* su,
                            const float* si, int D, float mu, float alpha, float beta,
                            int hot_T, int cpw, float flush_scale, int blocks, double* sse,
                            int variant, const unsigned int* packed, const int* chdr,
                            const float* rtable, cudaStream_t stream) {
  if (nnz <= 0) return 0;
  if (nnz % 32 != 0 || hot_T < 0) return (int)cudaErrorInvalidValue;
  MfArgs a;
  a.ru = ru; a.ri = ri; a.rr = rr; a.nnz = nnz;
  a.W = W; a.H = H; a.bu = bu; a.bi = bi; a.su = su; a.si = si;
  a.mu = mu; a.alpha = alpha; a.beta = beta;
  a.nchunks = nnz / 32;
  a.stride = 1;
  a.sse = sse;
  a.packed = packed; a.chdr = chdr; a.rtable = rtable;
  if (packed != nullptr && (chdr == nullptr || rtable == nullptr || variant == 2))
    return (int)cudaErrorInvalidValue;
  a.hot_T = hot_T;
  a.cpw = cpw > 0 ? cpw : 8;
  const int threads = 512;
  const bool g8 = (D == 128 && variant == 2);   // variant 2 selects the 8-lanes-per-rating kernel
  if (blocks <= 0) blocks = g8 ? 148 : 148 * 2;
  const int units = g8 ? (threads / 32) * 4 : (threads / 32);  // chunks in flight per CTA
  long long need = (a.nchunks + units - 1) / units;
  if (need < blocks) blocks = (int)need;
  a.flush_scale = flush_scale > 0.f ? flush_scale : 1.f / (float)blocks;
  size_t smem = (size_t)hot_T * (2 * (size_t)D + 2) * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (g8) {
    smem = (size_t)hot_T * (2 * (size_t)G8_STRIDE + 2) * sizeof(float);
    if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
    e = cudaFuncSetAttribute(mf_sgd_kernel_g8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    mf_sgd_kernel_g8<<<blocks, threads, smem, stream>>>(a);
    return pcl_last_error();
  }
  if (smem > 110 * 1024) return (int)cudaErrorInvalidValue;
  switch (D) {
    case 32:
      e = cudaFuncSetAttribute(mf_sgd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) mf_sgd_kernel<1><<<blocks, threads, smem, stream>>>(a);
      break;
    case 64:
      e = cudaFuncSetAttribute(mf_sgd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) mf_sgd_kernel<2><<<blocks, threads, smem, stream>>>(a);
      break;
    case 128:
      e = cudaFuncSetAttribute(mf_sgd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) mf_sgd_kernel<4><<<blocks, threads, smem, stream>>>(a);
      break;
    case 256:
      e = cudaFuncSetAttribute(mf_sgd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess) mf_sgd_kernel<8><<<blocks, threads, smem, stream>>>(a);
      break;
    default: return (int)cudaErrorInvalidValue;
  }
  if (e != cudaSuccess) return (int)e;
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
