// MF-SGD pass, rank 128, sixteen lanes per rating: a warp advances TWO chunks of 32
// ratings at once, one per half-warp, and a lane keeps 8 floats of every 128-float row
// (elements h*64 + l*4 + t, h < 2, t < 4: two 128-bit loads, each covering 256 contiguous
// bytes per half-warp).  One warp-wide instruction therefore serves two ratings, which
// roughly halves the instructions per rating of the 32-lanes-per-rating kernel in mf.cu
// (that kernel is bound by instruction issue, not by memory).  Everything else is the same
// algorithm (alg/recommendation/matrix_factorization/mf.hpp:266-280 for the update rule,
// 217-262 for the mixing weights): user row in registers while the chunk stays on one user,
// cold item rows read with L1-bypassing loads and updated with vector reductions, the
// hottest item rows replicated in shared memory per CTA and mixed into the global rows
// every `cpw` chunks, compact or plain rating stream.
//
// Hot replicas are kept as a float base value plus a 32-bit fixed-point delta (2^-22 units):
// the deltas are accumulated with native integer shared-memory atomics, which neither spin nor
// retry under contention the way a floating-point shared-memory atomic add does.
#include "common.cuh"

namespace {

struct MfH16Args {
  const int* ru;
  const int* ri;
  const float* rr;
  long long nnz;
  float* W;
  float* H;
  float* bu;
  float* bi;
  const float* su;
  const float* si;
  float mu, alpha, beta;
  long long nchunks;
  double* sse;
  int hot_T;
  int cpw;
  float flush_scale;
  const unsigned int* packed;
  const int* chdr;
  const float* rtable;
  const float* hot_fs;   // per hot row: weight of a CTA's delta in the mix (null: flush_scale)
  int packed_bits;       // 32: one word per rating (item | code << 24); 24: three bytes per rating
                         // (item | code << 21), 24 words per chunk of 32 ratings
};

struct Row8 {
  float4 a, b;   // elements l*4 .. l*4+3 and 64 + l*4 .. 64 + l*4 + 3
};

__device__ __forceinline__ Row8 load_cg(const float* row, int l) {
  Row8 r;
  r.a = pcl_ldcg4(row + l * 4);
  r.b = pcl_ldcg4(row + 64 + l * 4);
  return r;
}

// Packed pairs of fp32: sm_100 executes fma / mul / add on two fp32 values held in a 64-bit
// register pair as ONE instruction (fma.rn.f32x2 ...).  The pass is bound by instruction issue, so
// the element-wise parts of a rating (dot product, the two axpys, the fixed-point conversions'
// scaling) are written on pairs: half the floating-point instructions for the same arithmetic.
__device__ __forceinline__ unsigned long long pk2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void upk2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

constexpr float FX_SCALE = 4194304.f;          // 2^22
constexpr float FX_INV = 1.f / 4194304.f;

// Layout of a hot row's fixed-point deltas in shared memory.  Lane l of a half-warp owns elements
// 4 l + j and 64 + 4 l + j (j < 4) of a row; its j-th delta lives at word 16 j + l (64 + 16 j + l
// for the second group), so the sixteen lanes of one atomic instruction hit sixteen consecutive
// banks instead of every fourth one (a two-way conflict inside the half-warp and four-way when
// both halves update hot rows).  Rows are 144 words apart: consecutive rows start sixteen banks
// apart, so two hot rows of different parity do not collide either.
constexpr int HDS = 144;
__device__ __forceinline__ int hd_index(int idx) {   // idx = row * 128 + element
  const int e = idx & 127;
  return (idx >> 7) * HDS + (e & 64) + ((e & 3) << 4) + ((e & 63) >> 2);
}

// current value of a hot row: base + fixed-point delta
__device__ __forceinline__ Row8 load_hot(const float* base_row, const int* delta_row, int l) {
  const float4 b0 = *reinterpret_cast<const float4*>(base_row + l * 4);
  const float4 b1 = *reinterpret_cast<const float4*>(base_row + 64 + l * 4);
  const int4 d0 = make_int4(delta_row[l], delta_row[16 + l], delta_row[32 + l], delta_row[48 + l]);
  const int4 d1 = make_int4(delta_row[64 + l], delta_row[80 + l], delta_row[96 + l], delta_row[112 + l]);
  Row8 r;
  const unsigned long long inv2 = pk2(FX_INV, FX_INV);
  upk2(fma2(pk2((float)d0.x, (float)d0.y), inv2, pk2(b0.x, b0.y)), r.a.x, r.a.y);
  upk2(fma2(pk2((float)d0.z, (float)d0.w), inv2, pk2(b0.z, b0.w)), r.a.z, r.a.w);
  upk2(fma2(pk2((float)d1.x, (float)d1.y), inv2, pk2(b1.x, b1.y)), r.b.x, r.b.y);
  upk2(fma2(pk2((float)d1.z, (float)d1.w), inv2, pk2(b1.z, b1.w)), r.b.z, r.b.w);
  return r;
}

__device__ __forceinline__ void red_global(float* row, int l, const Row8& d) {
  pcl_red_add4(row + l * 4, d.a);
  pcl_red_add4(row + 64 + l * 4, d.b);
}

__device__ __forceinline__ int to_fx(float x) { return __float2int_rn(x * FX_SCALE); }

__device__ __forceinline__ void add_hot(int* row, int l, const Row8& d) {
  int* p = row + l;
  const unsigned long long sc2 = pk2(FX_SCALE, FX_SCALE);
  float x0, x1, x2, x3, x4, x5, x6, x7;
  upk2(mul2(pk2(d.a.x, d.a.y), sc2), x0, x1);
  upk2(mul2(pk2(d.a.z, d.a.w), sc2), x2, x3);
  upk2(mul2(pk2(d.b.x, d.b.y), sc2), x4, x5);
  upk2(mul2(pk2(d.b.z, d.b.w), sc2), x6, x7);
  atomicAdd(p, __float2int_rn(x0)); atomicAdd(p + 16, __float2int_rn(x1));
  atomicAdd(p + 32, __float2int_rn(x2)); atomicAdd(p + 48, __float2int_rn(x3));
  atomicAdd(p + 64, __float2int_rn(x4)); atomicAdd(p + 80, __float2int_rn(x5));
  atomicAdd(p + 96, __float2int_rn(x6)); atomicAdd(p + 112, __float2int_rn(x7));
}

__device__ __forceinline__ float dot8(const Row8& x, const Row8& y) {
  unsigned long long s = mul2(pk2(x.a.x, x.a.y), pk2(y.a.x, y.a.y));
  s = fma2(pk2(x.a.z, x.a.w), pk2(y.a.z, y.a.w), s);
  s = fma2(pk2(x.b.x, x.b.y), pk2(y.b.x, y.b.y), s);
  s = fma2(pk2(x.b.z, x.b.w), pk2(y.b.z, y.b.w), s);
  float lo, hi;
  upk2(s, lo, hi);
  return lo + hi;
}

// out = p * x + q * y, element-wise
__device__ __forceinline__ Row8 axpby(float p, const Row8& x, float q, const Row8& y) {
  Row8 o;
  const unsigned long long p2 = pk2(p, p), q2 = pk2(q, q);
  upk2(fma2(p2, pk2(x.a.x, x.a.y), mul2(q2, pk2(y.a.x, y.a.y))), o.a.x, o.a.y);
  upk2(fma2(p2, pk2(x.a.z, x.a.w), mul2(q2, pk2(y.a.z, y.a.w))), o.a.z, o.a.w);
  upk2(fma2(p2, pk2(x.b.x, x.b.y), mul2(q2, pk2(y.b.x, y.b.y))), o.b.x, o.b.y);
  upk2(fma2(p2, pk2(x.b.z, x.b.w), mul2(q2, pk2(y.b.z, y.b.w))), o.b.z, o.b.w);
  return o;
}

__device__ __forceinline__ void add_to(Row8& x, const Row8& d) {
  x.a.x += d.a.x; x.a.y += d.a.y; x.a.z += d.a.z; x.a.w += d.a.w;
  x.b.x += d.b.x; x.b.y += d.b.y; x.b.z += d.b.z; x.b.w += d.b.w;
}

__device__ __forceinline__ Row8 scaled_diff(float s, const Row8& x, const Row8& y) {
  Row8 o;
  o.a.x = s * (x.a.x - y.a.x); o.a.y = s * (x.a.y - y.a.y); o.a.z = s * (x.a.z - y.a.z);
  o.a.w = s * (x.a.w - y.a.w);
  o.b.x = s * (x.b.x - y.b.x); o.b.y = s * (x.b.y - y.b.y); o.b.z = s * (x.b.z - y.b.z);
  o.b.w = s * (x.b.w - y.b.w);
  return o;
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS, 1) mf_sgd_kernel_h16(MfH16Args a) {
  constexpr int D = 128;
  extern __shared__ float smem[];
  const int T = a.hot_T;
  int* hd = reinterpret_cast<int*>(smem);                   // T rows of fixed-point deltas (hd_index)
  float* hbase = smem + (size_t)T * HDS;                    // T x 128 values at the start of the period
  int* hbd = reinterpret_cast<int*>(hbase + (size_t)T * D); // T bias deltas
  float* hbb = reinterpret_cast<float*>(hbd + T);           // T bias bases
  const int lane = threadIdx.x & 31;
  const int g = lane >> 4;             // half-warp
  const int l = lane & 15;
  // the two half-warps take different branches (padding, user switch, hot or cold item), so every
  // shuffle names only the 16 lanes of its own half
  const unsigned gmask = 0xffffu << (16 * g);
  const int gic = (threadIdx.x >> 5) * 2 + g;   // half-warp index within the CTA
  const int gpc = (blockDim.x >> 5) * 2;
  const float ab = a.alpha * a.beta;
  const float keep = 1.f - ab;
  float sse = 0.f;

  const long long cta_chunks = a.nchunks > blockIdx.x
      ? (a.nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const long long iters = (cta_chunks + gpc - 1) / gpc;

  for (long long it = 0; it < iters; ++it) {
    if (T > 0 && (it % a.cpw) == 0) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
        float* gp = a.H + idx;           // hot rows are the first T rows of H
        const int hx = hd_index(idx);
        if (it > 0) {
          const int d = hd[hx];
          if (d != 0) atomicAdd(gp, (float)d * (FX_INV * (a.hot_fs ? a.hot_fs[idx >> 7] : a.flush_scale)));
        }
        hd[hx] = 0;
        hbase[idx] = __ldcg(gp);
      }
      for (int row = threadIdx.x; row < T; row += blockDim.x) {
        if (it > 0) {
          const int d = hbd[row];
          if (d != 0) atomicAdd(a.bi + row, (float)d * (FX_INV * (a.hot_fs ? a.hot_fs[row] : a.flush_scale)));
        }
        hbd[row] = 0;
        hbb[row] = __ldcg(a.bi + row);
      }
      __syncthreads();
    }
    const long long c = (long long)blockIdx.x + ((long long)gic + it * gpc) * gridDim.x;
    const bool live = c < a.nchunks;     // uniform per half-warp; a dead half sees only padding
    const long long base = c * 32;
    // entries l and l + 16 of this half-warp's chunk
    int u0 = -1, u1 = -1, i0 = 0, i1 = 0;
    float r0 = 0.f, r1 = 0.f;
    if (live) {
      if (a.packed != nullptr) {
        unsigned int pk0, pk1;
        if (a.packed_bits == 24) {
          // 24 words per chunk: lane l of the half-warp holds words l and (l < 8) 16 + l; entry e
          // starts at bit 24 e, i.e. in word (3 e) >> 2 at shift 8 * ((3 e) & 3)
          const unsigned int* cw = a.packed + c * 24;
          const unsigned int wa = __ldg(cw + l);
          const unsigned int wb = l < 8 ? __ldg(cw + 16 + l) : 0u;
          const int q0 = (3 * l) >> 2, q1 = (3 * (l + 16)) >> 2;          // q0 <= 11, 12 <= q1 <= 23
          const int src_base = g << 4;
          const unsigned int lo0 = __shfl_sync(gmask, wa, src_base + q0);
          const unsigned int hi0 = __shfl_sync(gmask, wa, src_base + q0 + 1);   // q0 + 1 <= 12
          const unsigned int a1 = __shfl_sync(gmask, wa, src_base + (q1 & 15));
          const unsigned int b1 = __shfl_sync(gmask, wb, src_base + (q1 & 15));
          const unsigned int a2 = __shfl_sync(gmask, wa, src_base + ((q1 + 1) & 15));
          const unsigned int b2 = __shfl_sync(gmask, wb, src_base + ((q1 + 1) & 15));
          const unsigned int lo1 = q1 < 16 ? a1 : b1;
          const unsigned int hi1 = (q1 + 1) < 16 ? a2 : b2;   // word 24 (q1 = 23) is never needed: its lane reads 0
          const unsigned int v0 = __funnelshift_r(lo0, hi0, 8 * ((3 * l) & 3)) & 0xffffffu;
          const unsigned int v1 = __funnelshift_r(lo1, hi1, 8 * ((3 * (l + 16)) & 3)) & 0xffffffu;
          pk0 = (v0 & 0x1fffffu) | ((v0 >> 21) << 24);
          pk1 = (v1 & 0x1fffffu) | ((v1 >> 21) << 24);
        } else {
          pk0 = __ldg(a.packed + base + l);
          pk1 = __ldg(a.packed + base + 16 + l);
        }
        const int u_base = __ldg(a.chdr + 3 * c);
        const unsigned int inc = (unsigned int)__ldg(a.chdr + 3 * c + 1);
        const int n_valid = __ldg(a.chdr + 3 * c + 2);
        i0 = (int)(pk0 & 0xffffffu);
        i1 = (int)(pk1 & 0xffffffu);
        r0 = __ldg(a.rtable + (pk0 >> 24));
        r1 = __ldg(a.rtable + (pk1 >> 24));
        u0 = l < n_valid ? u_base + __popc(inc & (0xffffffffu >> (31 - l))) : -1;
        u1 = l + 16 < n_valid ? u_base + __popc(inc & (0xffffffffu >> (15 - l))) : -1;
      } else {
        u0 = __ldg(a.ru + base + l);       u1 = __ldg(a.ru + base + 16 + l);
        i0 = __ldg(a.ri + base + l);       i1 = __ldg(a.ri + base + 16 + l);
        r0 = __ldg(a.rr + base + l);       r1 = __ldg(a.rr + base + 16 + l);
      }
    }
    int cur_u = -1;
    Row8 w, w0;
    w.a = w.b = w0.a = w0.b = make_float4(0.f, 0.f, 0.f, 0.f);
    float bu = 0.f, bu0 = 0.f, s_u = 1.f;

    const int src0 = g << 4;   // first lane of this half-warp
    int i_nxt = __shfl_sync(gmask, i0, src0);
    float si_nxt = __ldg(a.si + i_nxt);
    Row8 h_nxt;
    h_nxt.a = h_nxt.b = make_float4(0.f, 0.f, 0.f, 0.f);
    float bi_nxt = 0.f;
    if (i_nxt >= T) {
      h_nxt = load_cg(a.H + (long long)i_nxt * D, l);
      bi_nxt = __ldcg(a.bi + i_nxt);
    }

#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
      const int src = src0 + (j & 15);
      const int u = __shfl_sync(gmask, j < 16 ? u0 : u1, src);
      const float r = __shfl_sync(gmask, j < 16 ? r0 : r1, src);
      const int i = i_nxt;
      const bool hot = i < T;
      Row8 h = h_nxt;
      float bi = bi_nxt;
      const float s_i = si_nxt;
      const bool more = j + 1 < 32;
      if (more) {
        const int srcn = src0 + ((j + 1) & 15);
        i_nxt = __shfl_sync(gmask, j + 1 < 16 ? i0 : i1, srcn);
        si_nxt = __ldg(a.si + i_nxt);
        if (i_nxt >= T) {
          h_nxt = load_cg(a.H + (long long)i_nxt * D, l);
          bi_nxt = __ldcg(a.bi + i_nxt);
        }
      }
      if (u < 0) continue;   // padding (uniform per half-warp)
      if (hot) {
        h = load_hot(hbase + i * D, hd + i * HDS, l);
        bi = fmaf((float)hbd[i], FX_INV, hbb[i]);
      }
      if (u != cur_u) {
        if (cur_u >= 0) {
          red_global(a.W + (long long)cur_u * D, l, scaled_diff(s_u, w, w0));
          if (l == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
        }
        cur_u = u;
        w = load_cg(a.W + (long long)u * D, l);
        w0 = w;
        bu = __ldcg(a.bu + u);
        bu0 = bu;
        s_u = __ldg(a.su + u);
      }
      float dot = dot8(w, h);
      dot += __shfl_xor_sync(gmask, dot, 8);
      dot += __shfl_xor_sync(gmask, dot, 4);
      dot += __shfl_xor_sync(gmask, dot, 2);
      dot += __shfl_xor_sync(gmask, dot, 1);
      float pred = a.mu + bu + bi + dot;
      pred = fminf(5.f, fmaxf(1.f, pred));
      const float e = r - pred;
      sse = fmaf(e, e, sse);
      const float a2e = 2.f * a.alpha * e;
      // dH = s_i (a2e W - ab H), W <- (1 - ab) W + a2e H   (both from the pre-update values)
      const Row8 dh = axpby(s_i * a2e, w, -s_i * ab, h);
      w = axpby(keep, w, a2e, h);
      const float dbi = s_i * (a2e - ab * bi);
      bu += a2e - ab * bu;
      if (hot) {
        add_hot(hd + i * HDS, l, dh);
        if (l == 0) atomicAdd(&hbd[i], to_fx(dbi));
      } else {
        red_global(a.H + (long long)i * D, l, dh);
        if (l == 0) atomicAdd(a.bi + i, dbi);
        if (more && i_nxt == i) {   // the prefetched copy predates this update
          add_to(h_nxt, dh);
          bi_nxt += dbi;
        }
      }
    }
    if (cur_u >= 0) {
      red_global(a.W + (long long)cur_u * D, l, scaled_diff(s_u, w, w0));
      if (l == 0) atomicAdd(a.bu + cur_u, s_u * (bu - bu0));
    }
  }
  if (T > 0) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < T * D; idx += blockDim.x) {
      const int d = hd[hd_index(idx)];
      if (d != 0) atomicAdd(a.H + idx, (float)d * (FX_INV * (a.hot_fs ? a.hot_fs[idx >> 7] : a.flush_scale)));
    }
    for (int row = threadIdx.x; row < T; row += blockDim.x) {
      const int d = hbd[row];
      if (d != 0) atomicAdd(a.bi + row, (float)d * (FX_INV * (a.hot_fs ? a.hot_fs[row] : a.flush_scale)));
    }
  }
  if (a.sse != nullptr && l == 0 && sse != 0.f) atomicAdd(a.sse, (double)sse);
}

}  // namespace

// Same contract as pcl_mf_sgd_pass (mf.cu) for D = 128: user-major sorted ratings in chunks of
// 32, plain (ru, ri, rr) or compact (packed, chdr, rtable) stream, hot item rows (local index
// below hot_T) replicated in shared memory and mixed every `cpw` chunks per half-warp with
// weight `flush_scale` (<= 0: 1 / blocks) or, when `hot_fs` is given, with one weight per hot row.
// `packed_bits` 24 selects the three-bytes-per-rating stream (21-bit item index, 3-bit rating code).  `blocks` <= 0 selects one CTA per SM; `threads` is 512, 640 (default), 768 or 1024
// (threads / 16 chunks in flight per CTA).
PCL_API int pcl_mf_sgd_pass_h16(const int* ru, const int* ri, const float* rr, long long nnz,
                                float* W, float* H, float* bu, float* bi, const float* su,
                                const float* si, float mu, float alpha, float beta, int hot_T,
                                int cpw, float flush_scale, int blocks, double* sse,
                                const unsigned int* packed, const int* chdr, const float* rtable,
                                int threads, const float* hot_fs, int packed_bits, cudaStream_t stream) {
  if (nnz <= 0) return 0;
  if (nnz % 32 != 0 || hot_T < 0) return (int)cudaErrorInvalidValue;
  if (packed != nullptr && (chdr == nullptr || rtable == nullptr)) return (int)cudaErrorInvalidValue;
  if (packed == nullptr && (ru == nullptr || ri == nullptr || rr == nullptr))
    return (int)cudaErrorInvalidValue;
  MfH16Args a;
  a.ru = ru; a.ri = ri; a.rr = rr; a.nnz = nnz;
  a.W = W; a.H = H; a.bu = bu; a.bi = bi; a.su = su; a.si = si;
  a.mu = mu; a.alpha = alpha; a.beta = beta;
  a.nchunks = nnz / 32;
  a.sse = sse;
  a.hot_T = hot_T;
  a.cpw = cpw > 0 ? cpw : 8;
  a.packed = packed; a.chdr = chdr; a.rtable = rtable;
  a.hot_fs = hot_fs;
  if (packed != nullptr && packed_bits != 24 && packed_bits != 32) return (int)cudaErrorInvalidValue;
  a.packed_bits = packed_bits;
  if (threads <= 0) threads = 640;   // 20 warps = 40 chunks in flight per CTA
  if (threads != 512 && threads != 640 && threads != 768 && threads != 1024) return (int)cudaErrorInvalidValue;
  if (blocks <= 0) blocks = 148;
  const int per_cta = threads / 16;
  const long long need = (a.nchunks + per_cta - 1) / per_cta;
  if (need < blocks) blocks = (int)need;
  a.flush_scale = flush_scale > 0.f ? flush_scale : 1.f / (float)blocks;
  const size_t smem = (size_t)hot_T * (HDS + 128 + 2) * sizeof(float);
  if (smem > 220 * 1024) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
#define PCL_H16_LAUNCH(T)                                                                              \
  e = cudaFuncSetAttribute(mf_sgd_kernel_h16<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
  if (e == cudaSuccess) mf_sgd_kernel_h16<T><<<blocks, T, smem, stream>>>(a);
  switch (threads) {
    case 512: PCL_H16_LAUNCH(512) break;
    case 640: PCL_H16_LAUNCH(640) break;
    case 768: PCL_H16_LAUNCH(768) break;
    default: PCL_H16_LAUNCH(1024) break;
  }
#undef PCL_H16_LAUNCH
  if (e != cudaSuccess) return (int)e;
  return pcl_last_error();
}
