// C[M x N] = A[M x K] * B[N x K]^T in fp32 storage on the 5th-generation tensor
// cores (tcgen05.mma kind::tf32, fp32 accumulators in tensor memory), with the
// all-gather of a sharded B fused in ("dense paracel_read" of a parameter that
// is range-sharded over the ranks, followed by the first GEMM that consumes
// it; reference call sites: paracel_read("clusters_k") + the distance loop of
// alg/clustering/kmeans/kmeans.hpp:113-133, the all-pairs dot products of
// alg/recommendation/similarity_dense/sim_dense.hpp:84-101).
//
// Structure of one persistent CTA (192 threads, one CTA per SM):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D loads of a 128 x 32 A tile
//               and a 128 x 32 B tile per stage (128-byte swizzle), 6 stages
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M128 N128 K8)
//               and commits to mbarriers
//   warps 2-5   epilogue: tcgen05.ld of the 128 x 128 accumulator (two buffers, so
//               the MMAs of the next tile overlap), then either a row-major store
//               or a running row-wise argmin of (bnorm[n] - 2 * acc) (k-means)
// Work unit = one 128-row block of A; the CTA walks all column tiles of B for it,
// starting with the tiles owned by this rank.
//
// Fused gather (world > 1): the first `gather_ctas` CTAs copy the peers' shards
// of B into a local staging buffer with 128-bit peer loads, tile by tile, and
// release a flag per tile; the producer warp waits (bounded) on the flag and
// then issues an ordinary TMA load from LOCAL memory.  No TMA load ever touches
// peer memory and no load uses cluster multicast.
//
// Every wait (mbarrier or flag) is bounded; on expiry the kernel records a
// status, every role leaves its loops, tensor memory is freed and the kernel
// returns.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 32;       // 32 fp32 = 128 bytes = one swizzle row
constexpr int STAGES = 6;
constexpr int UMMA_K = 8;    // tf32
constexpr int A_BYTES = BM * BK * 4;
constexpr int B_BYTES = BN * BK * 4;
constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 256 /*barriers*/ +
                           4 * BN * 4 /*|b_n|^2 of the current tile, per epilogue warp*/;
constexpr unsigned SPIN_LIMIT = 1u << 24;

struct GemmArgs {
  float* C;            // M x N row-major (epi 0), may be null
  long long ldc;
  int M, N, K;
  int epi;             // 0 store, 1 row argmin of (bnorm[n] - 2 acc)
  const float* bnorm;  // N (epi 1)
  float* row_min;      // M (epi 1)
  int* row_arg;        // M (epi 1)
  // fused gather
  const float* const* b_shards;  // world base pointers, shard r holds rows [r*rps, (r+1)*rps)
  float* b_stage;                // N x K local staging (the TMA map of B points here)
  int* flags;                    // one per column tile
  int world, rank, rows_per_shard, epoch, gather_ctas;
  PclStatus* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait: false when the limit ran out or another role raised `abort`.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 63) == 63) {
      if (*abort_flag) return false;
      __nanosleep(64);
    }
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  // K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart
  const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);              // LBO = 1 (unused)
  const uint32_t hi = 64u /*SBO = 1024 B*/ | (1u << 14) /*version*/ | (2u << 29) /*SW128*/;
  return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void report(PclStatus* st, int rank, int wait_id, long long expected,
                                       long long seen) {
  if (st != nullptr && atomicCAS(&st->code, 0, 1) == 0) {
    st->rank = rank;
    st->wait_id = wait_id;
    st->expected = expected;
    st->seen = seen;
  }
}

// column tile visited at position `ord`: this rank's tiles first, then the peers' in ring order
__device__ __forceinline__ int tile_at(int ord, int n_tiles, int first_local) {
  int t = first_local + ord;
  return t >= n_tiles ? t - n_tiles : t;
}

__global__ void __launch_bounds__(192, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (a.N + BN - 1) / BN;
  const int m_tiles = (a.M + BM - 1) / BM;
  const int kb_count = (a.K + BK - 1) / BK;
  // tiles owned by this rank come first
  int first_local = 0;
  if (a.world > 1) first_local = (int)(((long long)a.rank * a.rows_per_shard) / BN) % n_tiles;

  // ------------------------------------------------------------ gather CTAs
  if ((int)blockIdx.x < a.gather_ctas) {
    const int kv = a.K >> 2;  // float4 per row (K % 4 == 0)
    for (int ord = blockIdx.x; ord < n_tiles; ord += a.gather_ctas) {
      const int nt = tile_at(ord, n_tiles, first_local);
      const int r0 = nt * BN;
      const int r1 = min(a.N, r0 + BN);
      // eight 128-bit peer loads in flight per thread before the first store
      const long long total = (long long)(r1 - r0) * kv;
      for (long long base = threadIdx.x; base < total; base += (long long)blockDim.x * 8) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const long long idx = base + (long long)u * blockDim.x;
          if (idx < total) {
            const int row = r0 + (int)(idx / kv);
            const int c = (int)(idx % kv);
            const int owner = min(row / a.rows_per_shard, a.world - 1);
            v[u] = pcl_ld_sys4(a.b_shards[owner] + (long long)(row - owner * a.rows_per_shard) * a.K + 4 * c);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const long long idx = base + (long long)u * blockDim.x;
          if (idx < total) {
            const int row = r0 + (int)(idx / kv);
            const int c = (int)(idx % kv);
            *reinterpret_cast<float4*>(a.b_stage + (long long)row * a.K + 4 * c) = v[u];
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(a.flags + nt), "r"(a.epoch) : "memory");
      }
    }
    return;
  }

  // --------------------------------------------------------------- MMA CTAs
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + STAGES * A_BYTES;
  uint64_t* bars = (uint64_t*)(base + STAGES * (A_BYTES + B_BYTES));
  uint64_t* full = bars;                 // STAGES
  uint64_t* empty = bars + STAGES;       // STAGES
  uint64_t* tfull = bars + 2 * STAGES;   // 2
  uint64_t* tempty = tfull + 2;          // 2
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull + b, 1); mbar_init(tempty + b, 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int cta = (int)blockIdx.x - a.gather_ctas;
  const int ncta = (int)gridDim.x - a.gather_ctas;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int mt = cta; mt < m_tiles && ok; mt += ncta) {
        for (int ord = 0; ord < n_tiles && ok; ++ord) {
          const int nt = tile_at(ord, n_tiles, first_local);
          if (a.gather_ctas > 0) {  // bounded wait for the staged column tile
            int seen = 0;
            unsigned it = 0;
            for (; it < SPIN_LIMIT; ++it) {
              seen = pcl_ld_acquire_sys_i32(a.flags + nt);
              if (seen == a.epoch) break;
              if (*abort_flag) break;
              __nanosleep(128);
            }
            if (seen != a.epoch) {
              report(a.status, a.rank, 10, a.epoch, seen);
              *abort_flag = 1;
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");  // staged by generic stores, read by TMA
          }
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(empty + stage, phase ^ 1, abort_flag)) {
              report(a.status, a.rank, 11, kb, stage);
              *abort_flag = 1;
              ok = false;
              break;
            }
            mbar_expect_tx(full + stage, A_BYTES + B_BYTES);
            tma_load_2d(sA + stage * A_BYTES, &tmA, full + stage, kb * BK, mt * BM);
            tma_load_2d(sB + stage * B_BYTES, &tmB, full + stage, kb * BK, nt * BN);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight time to land before shared memory goes away
        for (int s = 0; s < 2048; ++s) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      for (int mt = cta; mt < m_tiles && ok; mt += ncta) {
        for (int ord = 0; ord < n_tiles && ok; ++ord) {
          if (!mbar_wait(tempty + acc, acc_phase[acc] ^ 1, abort_flag)) {
            report(a.status, a.rank, 12, acc, 0);
            *abort_flag = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t d = tmem_base + (uint32_t)(acc * BN);
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(full + stage, phase, abort_flag)) {
              report(a.status, a.rank, 13, kb, stage);
              *abort_flag = 1;
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = make_desc_sw128(smem_u32(sA + stage * A_BYTES));
            const uint64_t db = make_desc_sw128(smem_u32(sB + stage * B_BYTES));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // +32 bytes along K inside the swizzle row = +2 in the encoded address
              umma_tf32(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(empty + stage);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(tfull + acc);
          acc_phase[acc] ^= 1;
          acc ^= 1;
        }
      }
    }
  } else {
    // epilogue warps 2..5; a warp may only touch the 32 TMEM lanes of its sub-partition
    const int sub = warp & 3;
    const int row_in_tile = sub * 32 + lane;
    float* bn_s = reinterpret_cast<float*>(base + STAGES * (A_BYTES + B_BYTES) + 256) + (warp - 2) * BN;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    for (int mt = cta; mt < m_tiles && ok; mt += ncta) {
      const int row = mt * BM + row_in_tile;
      float best = 3.402823466e38f;
      int best_n = 0;
      for (int ord = 0; ord < n_tiles && ok; ++ord) {
        const int nt = tile_at(ord, n_tiles, first_local);
        if (!mbar_wait(tfull + acc, acc_phase[acc], abort_flag)) {
          if (lane == 0) report(a.status, a.rank, 14, acc, 0);
          *abort_flag = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t0 = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(acc * BN);
        if (a.epi == 1) {   // |b_n|^2 of this tile's columns, +inf beyond N
          __syncwarp();
          for (int q = lane; q < BN; q += 32) {
            const int n = nt * BN + q;
            bn_s[q] = n < a.N ? __ldg(a.bnorm + n) : 3.402823466e38f;
          }
          __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld32(t0 + (uint32_t)(c * 32), v);
          const int n0 = nt * BN + c * 32;
          if (a.epi == 0) {
            if (row < a.M) {
              float* dst = a.C + (long long)row * a.ldc + n0;
              if (n0 + 32 <= a.N && ((a.ldc & 3) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (n0 + j < a.N) dst[j] = v[j];
              }
            }
          } else {
            // dist[j] = |b_n|^2 - 2 a.b_n; the minimum first (one FMNMX per column), the column
            // index only when this chunk improves the running best, which becomes rare quickly
            float d[32];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 b = *reinterpret_cast<const float4*>(bn_s + c * 32 + 4 * q);
              d[4 * q] = fmaf(-2.f, v[4 * q], b.x);
              d[4 * q + 1] = fmaf(-2.f, v[4 * q + 1], b.y);
              d[4 * q + 2] = fmaf(-2.f, v[4 * q + 2], b.z);
              d[4 * q + 3] = fmaf(-2.f, v[4 * q + 3], b.w);
            }
            float m16[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) m16[j] = fminf(d[j], d[j + 16]);
#pragma unroll
            for (int w = 8; w >= 1; w >>= 1)
#pragma unroll
              for (int j = 0; j < w; ++j) m16[j] = fminf(m16[j], m16[j + w]);
            const float m = m16[0];
            if (m <= best) {
              int jn = 31;
#pragma unroll
              for (int j = 30; j >= 0; --j) jn = (d[j] == m) ? j : jn;
              const int n = n0 + jn;
              if (m < best || n < best_n) { best = m; best_n = n; }
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty + acc);
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
      if (ok && a.epi == 1 && row < a.M) {
        a.row_min[row] = best;
        a.row_arg[row] = best_n;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN));
  }
}

typedef CUresult (*encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                CUtensorMapFloatOOBfill);

encode_fn_t get_encode() {
  static encode_fn_t fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (encode_fn_t)p;
  }
  return fn;
}

// rows x K fp32 row-major matrix, box = 32 floats (128 B) x box_rows rows, 128-byte swizzle
int make_map(CUtensorMap* map, const float* ptr, long long rows, long long K, int box_rows) {
  encode_fn_t enc = get_encode();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)ptr, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace

// C = A * B^T with A [M x K], B [N x K] row-major fp32 (16-byte aligned, K % 4 == 0).
//   epi 0: C [M x N] with leading dimension ldc is written.
//   epi 1: row_min[m] = min_n (bnorm[n] - 2 * C[m][n]), row_arg[m] = its n (C is not written).
// Fused gather: when world > 1, `b_shards` is a device array of `world` pointers, shard r
// holding rows [r * rows_per_shard, ...) of B; the rows are staged into `b_stage` (N x K,
// local memory) by `gather_ctas` CTAs and `flags` (one int per 128-column tile, zero
// initialised once) is stamped with `epoch`, which the caller increases on every call.
// With world == 1 pass b_shards = null and b_stage = B.
// `status` (optional) receives the record of a wait that ran out.
PCL_API int pcl_gemm_tf32(const float* A, float* b_stage, float* C, int M, int N, int K,
                          long long ldc, int epi, const float* bnorm, float* row_min, int* row_arg,
                          const float* const* b_shards, int* flags, int world, int rank,
                          int rows_per_shard, int epoch, int gather_ctas, PclStatus* status,
                          int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 3) || ((uintptr_t)A & 15) || ((uintptr_t)b_stage & 15)) return (int)cudaErrorInvalidValue;
  if (epi == 0 && C == nullptr) return (int)cudaErrorInvalidValue;
  if (epi == 1 && (bnorm == nullptr || row_min == nullptr || row_arg == nullptr))
    return (int)cudaErrorInvalidValue;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, BM);
  if (rc) return rc;
  rc = make_map(&tmB, b_stage, N, K, BN);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.epi = epi;
  a.bnorm = bnorm; a.row_min = row_min; a.row_arg = row_arg;
  a.b_shards = b_shards; a.b_stage = b_stage; a.flags = flags;
  a.world = world; a.rank = rank; a.rows_per_shard = rows_per_shard > 0 ? rows_per_shard : N;
  a.epoch = epoch; a.status = status;
  if (num_sms <= 0) num_sms = 148;
  const bool fused = (world > 1 && b_shards != nullptr);
  a.gather_ctas = fused ? (gather_ctas > 0 ? gather_ctas : 16) : 0;
  if (fused && flags == nullptr) return (int)cudaErrorInvalidValue;
  const int m_tiles = (M + BM - 1) / BM;
  int mma_ctas = num_sms - a.gather_ctas;
  if (mma_ctas > m_tiles) mma_ctas = m_tiles;
  if (mma_ctas < 1) mma_ctas = 1;
  cudaError_t e = cudaFuncSetAttribute(gemm_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  gemm_tf32_kernel<<<a.gather_ctas + mma_ctas, 192, SMEM_BYTES, stream>>>(tmA, tmB, a);
  return pcl_last_error();
}

// Split x into a tf32-representable high part and the remainder, written K-concatenated so
// that one tf32 GEMM over 3K columns evaluates hi*hi + hi*lo + lo*hi (error-compensated
// "3xTF32", fp32-level accuracy):  a_out[m] = [hi | hi | lo],  b_out[n] = [hi | lo | hi].
__global__ void split3_kernel(const float* x, float* out, long long rows, int K, int is_b) {
  const long long total = rows * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / K;
    const int k = (int)(i % K);
    const float v = x[i];
    const float hi = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    const float lo = v - hi;
    float* o = out + r * 3 * K;
    o[k] = hi;
    o[K + k] = is_b ? lo : hi;
    o[2 * K + k] = is_b ? hi : lo;
  }
}

PCL_API int pcl_split3_tf32(const float* x, float* out, long long rows, int K, int is_b,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  long long total = rows * K;
  int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  split3_kernel<<<blocks, 256, 0, stream>>>(x, out, rows, K, is_b);
  return pcl_last_error();
}
