// Dense parameter vectors sharded by range over the ranks ("theta"-style keys).
//
//   dense_read     all-gather: every rank copies all shards into a local full
//                  vector with 128-bit peer loads (paracel_read of a dense key,
//                  reference include/ps.hpp:437-462 + one TCP round trip).
//   dense_bupdate  reduce-scatter fused with the registered update handler:
//                  the owner of a slice sums that slice of every rank's delta
//                  vector straight out of peer memory and applies
//                      add       theta += sum                    (lr_theta_update, default_incr_*)
//                      sgd       theta -= lr * sum
//                      prox_l1   w = theta - lr * sum; theta = sign(w) max(|w| - |lr|*lambda, 0)
//                      max       theta = max(theta, max_r delta_r)
//                  (paracel_bupdate + server-side handler, ps.hpp:779-798,
//                  include/server.hpp:88-100, 331-349).
//   publish        release-store of an epoch number into slot [rank] of every
//                  peer's flag array (delta ready / update done).
// Both kernels start with a bounded wait on a local flag array that the peers
// publish into; the last block of dense_bupdate publishes "done".
#include "common.cuh"

namespace {

enum DenseHandler { DH_ADD = 0, DH_SGD = 1, DH_PROX_L1 = 2, DH_MAX = 3 };

struct ReadArgs {
  const float* const* shards;  // world pointers, shard r = elements [r*S, (r+1)*S)
  float* out;                  // full vector, L floats
  long long L, S;
  int world, rank;
  const long long* flags;      // wait for min(flags[0..world)) >= target (null: no wait)
  long long target;
  unsigned long long timeout_ns;
  PclStatus* status;
};

__global__ void __launch_bounds__(256) dense_read_kernel(ReadArgs a) {
  __shared__ int ok;
  if (a.flags != nullptr && a.target > 0) {
    if (threadIdx.x == 0)
      ok = pcl_wait_min_clock(a.flags, a.world, a.target, a.timeout_ns, a.status, a.rank, 20) ? 1 : 0;
    __syncthreads();
    if (!ok) return;
  }
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  // Ring order: rank r copies its own shard first, then r + 1, r + 2, ...; at any moment the ranks
  // read from different owners instead of all from shard 0.  One loop per shard (no division to
  // find an element's owner), eight 16-byte loads in flight per thread.
  constexpr int U = 4;
  for (int k = 0; k < a.world; ++k) {
    int o = a.rank + k;
    if (o >= a.world) o -= a.world;
    const long long base = (long long)o * a.S;
    // the last shard takes whatever is left of L
    const long long len = (o == a.world - 1) ? a.L - base : (a.S < a.L - base ? a.S : a.L - base);
    if (len <= 0) continue;
    const float* src = a.shards[o];
    float* dst = a.out + base;
    const long long nv = len >> 2;
    for (long long v0 = tid; v0 < nv; v0 += U * nth) {
      float4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nth;
        if (v < nv) x[u] = pcl_ld_sys4(src + (v << 2));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nth;
        if (v < nv) *reinterpret_cast<float4*>(dst + (v << 2)) = x[u];
      }
    }
    for (long long e = (nv << 2) + tid; e < len; e += nth) dst[e] = src[e];
  }
}

struct BupArgs {
  float* theta;                 // this rank's shard, S floats (elements [rank*S, ...))
  const float* const* deltas;   // world pointers to full-length delta vectors (L floats each)
  long long L, S;
  int world, rank;
  int handler;
  float lr, lambda;
  const long long* ready;       // local flag array the peers publish "delta ready" into
  long long epoch;
  unsigned long long timeout_ns;
  PclStatus* status;
  long long* const* done_ptrs;  // world pointers to every rank's "done" array (may be null)
  unsigned int* block_counter;  // zero-initialised, reset by the last block
  double* nnz_out;              // optional: += number of non-zero entries of the new shard
};

__device__ __forceinline__ float apply_handler(int handler, float th, float sum, float mx, float lr,
                                               float lambda) {
  switch (handler) {
    case DH_ADD: return th + sum;
    case DH_SGD: return th - lr * sum;
    case DH_PROX_L1: {
      const float w = th - lr * sum;
      const float t = fabsf(lr) * lambda;  // lr may carry a sign / a 1/n factor of the caller's delta
      return w > t ? w - t : (w < -t ? w + t : 0.f);
    }
    default: return fmaxf(th, mx);
  }
}

// IS_MAX: the max handler keeps a running maximum of the deltas, every other handler their sum;
// the two forms are separate instances so that neither carries the other's registers.  Four
// 16-byte columns per thread: eight need 176 registers and were a quarter slower.
template <bool IS_MAX>
__global__ void __launch_bounds__(256) dense_bupdate_kernel(BupArgs a) {
  __shared__ int ok;
  if (a.ready != nullptr && a.epoch > 0) {
    if (threadIdx.x == 0)
      ok = pcl_wait_min_clock(a.ready, a.world, a.epoch, a.timeout_ns, a.status, a.rank, 21) ? 1 : 0;
    __syncthreads();
  }
  // After a timed-out wait the block does no work but still takes part in the block count below,
  // so that the counter is back at zero for the next launch; "done" is then not published.
  const bool proceed = !(a.ready != nullptr && a.epoch > 0) || ok;
  const long long lo = (long long)a.rank * a.S;
  long long n = a.L - lo;
  if (n > a.S) n = a.S;
  if (n < 0 || !proceed) n = 0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const bool vec_ok = ((lo & 3) == 0);
  const long long nvec = vec_ok ? (n >> 2) : 0;
  float nz = 0.f;
  // U independent 16-byte columns per thread and trip: all their loads (the shard and every
  // rank's delta) are issued before the first handler is applied
  constexpr int U = 2;
  for (long long v0 = tid; v0 < nvec; v0 += U * nth) {
    float4 s[U], t[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + u * nth;
      s[u] = IS_MAX ? make_float4(-3.4e38f, -3.4e38f, -3.4e38f, -3.4e38f) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < nvec) t[u] = *reinterpret_cast<const float4*>(a.theta + (v << 2));
    }
    for (int i = 0; i < a.world; ++i) {
      int r = a.rank + i;
      if (r >= a.world) r -= a.world;
      float4 d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * nth;
        if (v < nvec) d[u] = pcl_ld_sys4(a.deltas[r] + lo + (v << 2));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (v0 + u * nth >= nvec) continue;
        if (IS_MAX) {
          s[u].x = fmaxf(s[u].x, d[u].x); s[u].y = fmaxf(s[u].y, d[u].y);
          s[u].z = fmaxf(s[u].z, d[u].z); s[u].w = fmaxf(s[u].w, d[u].w);
        } else {
          s[u].x += d[u].x; s[u].y += d[u].y; s[u].z += d[u].z; s[u].w += d[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + u * nth;
      if (v >= nvec) continue;
      float4 x = t[u];
      x.x = apply_handler(a.handler, x.x, s[u].x, s[u].x, a.lr, a.lambda);
      x.y = apply_handler(a.handler, x.y, s[u].y, s[u].y, a.lr, a.lambda);
      x.z = apply_handler(a.handler, x.z, s[u].z, s[u].z, a.lr, a.lambda);
      x.w = apply_handler(a.handler, x.w, s[u].w, s[u].w, a.lr, a.lambda);
      *reinterpret_cast<float4*>(a.theta + (v << 2)) = x;
      nz += (x.x != 0.f) + (x.y != 0.f) + (x.z != 0.f) + (x.w != 0.f);
    }
  }
  for (long long e = (nvec << 2) + tid; e < n; e += nth) {
    float s = 0.f, m = -3.4e38f;
    for (int i = 0; i < a.world; ++i) {
      int r = a.rank + i;
      if (r >= a.world) r -= a.world;
      float d;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(d) : "l"(a.deltas[r] + lo + e));
      s += d;
      m = fmaxf(m, d);
    }
    const float t = apply_handler(a.handler, a.theta[e], s, m, a.lr, a.lambda);
    a.theta[e] = t;
    nz += (t != 0.f);
  }
  if (a.nnz_out != nullptr) {
    nz = pcl_warp_sum(nz);
    if ((threadIdx.x & 31) == 0 && nz != 0.f) atomicAdd(a.nnz_out, (double)nz);
  }
  // the last block to finish publishes "done" to every rank
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.block_counter, 1u);
    if (prev == gridDim.x - 1) {
      *a.block_counter = 0u;
      if (a.done_ptrs != nullptr && proceed) {
        __threadfence_system();
        for (int r = 0; r < a.world; ++r) pcl_st_release_sys(a.done_ptrs[r] + a.rank, a.epoch);
      }
    }
  }
}

// One-sided update of a dense key: this rank alone adds scale * delta into the owners' shards
// with vector reductions over NVLink (paracel_update / a bupdate with a linear handler that only
// one worker issues; include/ps.hpp:689-750).  Nothing waits and nothing is published.
struct PushDenseArgs {
  float* const* shards;
  const float* delta;   // L floats
  long long L, S;
  int world, rank;
  float scale;
};

__global__ void __launch_bounds__(256) dense_push_kernel(PushDenseArgs a) {
  const long long nvec = a.L >> 2;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const long long shift = nvec > 0 ? (((long long)a.rank * a.S) >> 2) % nvec : 0;
  for (long long v = tid; v < nvec; v += nth) {
    long long vv = v + shift;            // every rank starts at its own shard
    if (vv >= nvec) vv -= nvec;
    const long long e = vv << 2;
    float4 d = *reinterpret_cast<const float4*>(a.delta + e);
    d.x *= a.scale; d.y *= a.scale; d.z *= a.scale; d.w *= a.scale;
    if (d.x == 0.f && d.y == 0.f && d.z == 0.f && d.w == 0.f) continue;
    int owner = (int)(e / a.S);
    if (owner >= a.world) owner = a.world - 1;
    pcl_red_add4_sys(a.shards[owner] + (e - (long long)owner * a.S), d);
  }
  for (long long e = (nvec << 2) + tid; e < a.L; e += nth) {
    const float d = a.delta[e] * a.scale;
    if (d == 0.f) continue;
    int owner = (int)(e / a.S);
    if (owner >= a.world) owner = a.world - 1;
    asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(a.shards[owner] + (e - (long long)owner * a.S)),
                 "f"(d)
                 : "memory");
  }
}

__global__ void publish_kernel(long long* const* flag_ptrs, int world, int rank, long long value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    pcl_st_release_sys(flag_ptrs[r] + rank, value);
  }
}

}  // namespace

PCL_API int pcl_dense_read(const float* const* shards, float* out, long long L, long long S,
                           int world, int rank, const long long* flags, long long target,
                           unsigned long long timeout_ns, PclStatus* status, cudaStream_t stream) {
  if (L <= 0) return 0;
  if ((S & 3) && world > 1) return (int)cudaErrorInvalidValue;  // shards must keep 16-byte alignment
  ReadArgs a{shards, out, L, S, world, rank, flags, target, timeout_ns, status};
  long long blocks = (L / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dense_read_kernel<<<(int)blocks, 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_dense_bupdate(float* theta, const float* const* deltas, long long L, long long S,
                              int world, int rank, int handler, float lr, float lambda,
                              const long long* ready, long long epoch, unsigned long long timeout_ns,
                              PclStatus* status, long long* const* done_ptrs,
                              unsigned int* block_counter, double* nnz_out, cudaStream_t stream) {
  if (L <= 0) return 0;
  BupArgs a{theta, deltas, L, S, world, rank, handler, lr, lambda, ready, epoch, timeout_ns,
            status, done_ptrs, block_counter, nnz_out};
  long long blocks = (S / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (handler == DH_MAX) dense_bupdate_kernel<true><<<(int)blocks, 256, 0, stream>>>(a);
  else dense_bupdate_kernel<false><<<(int)blocks, 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_dense_push(float* const* shards, const float* delta, long long L, long long S,
                           int world, int rank, float scale, cudaStream_t stream) {
  if (L <= 0) return 0;
  if ((S & 3) && world > 1) return (int)cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(delta) & 15) return (int)cudaErrorInvalidValue;
  PushDenseArgs a{shards, delta, L, S, world, rank, scale};
  long long blocks = (L / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dense_push_kernel<<<(int)blocks, 256, 0, stream>>>(a);
  return pcl_last_error();
}

PCL_API int pcl_publish_flag(long long* const* flag_ptrs, int world, int rank, long long value,
                             cudaStream_t stream) {
  if (world > 1024) return (int)cudaErrorInvalidValue;
  publish_kernel<<<1, ((world + 31) / 32) * 32, 0, stream>>>(flag_ptrs, world, rank, value);
  return pcl_last_error();
}
