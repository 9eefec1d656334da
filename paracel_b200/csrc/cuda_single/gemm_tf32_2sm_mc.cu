// C[M x N] = A[M x K] * B[N x K]^T on one GPU: the two-CTA tcgen05 kernel of gemm_tf32_2sm.cu with
// clusters of FOUR CTAs (two pairs) that share their B operand through TMA multicast.
//
// The two pairs of a cluster work on vertically adjacent 256 x 256 tiles (rows 2 mt2 and 2 mt2 + 1,
// the same 256 columns).  CTA e of a pair needs rows [128 e, 128 e + 128) of the B tile; instead of
// both pairs fetching them, CTA e of pair j loads the 64 rows [128 e + 64 j, +64) once and the copy
// engine writes them into the shared memory of CTA e of BOTH pairs.  Per 32-deep K block a CTA then
// pulls 24 KB out of L2 (16 KB of A, 8 KB of B) instead of 32 KB, which is what limits the
// two-CTA kernel without multicast on the large shapes.
//
// Every operand of this kernel is memory of the launching GPU (plain device pointers passed by the
// caller; there is no shard table and no staging of peers' data here).  The file lives apart from
// the kernels that run on several GPUs, which use no multicast loads at all.
//
// Synchronisation differences from the pair kernel:
//   * a stage of CTA (j, e) is written by its own loads and by the B load of CTA (1 - j, e), so a
//     producer may refill a stage only when the MMAs of BOTH pairs have finished with it: the MMA
//     lane of each pair commits to the "empty" barrier of all four CTAs (tcgen05.commit with
//     multicast), and those barriers expect two arrivals;
//   * the bytes a CTA receives, whoever loaded them, are counted on the "full" barrier of the
//     leader of the RECEIVING pair (cta_group::2 form of the bulk tensor load);
//   * the two pairs therefore walk the K blocks of their tiles in lockstep; when the number of
//     256-row blocks is odd the second pair of the last cluster row multiplies rows beyond M
//     (zero-filled by the copy engine) and stores nothing.
// Every wait has a time limit; on expiry the status record is written, all four CTAs are told to
// leave, tensor memory is freed and the kernel ends.
#include <cuda.h>

#include "common.cuh"
#include "gemm_sm100.cuh"

namespace {

using namespace pcl_sm100;

constexpr int TM = 256;      // tile rows per CTA pair
constexpr int TN = 256;      // tile columns
constexpr int HM = 128;      // rows of A (and of the accumulator) per CTA
constexpr int HN = 128;      // rows of B per CTA
constexpr int QN = 64;       // rows of B a CTA loads itself (the other 64 come from the other pair)
constexpr int BK = 32;       // 32 fp32 = 128 bytes = one swizzle row
constexpr int STAGES = 6;
constexpr int UMMA_K = 8;
constexpr int A_BYTES = HM * BK * 4;
constexpr int B_BYTES = HN * BK * 4;
constexpr int Q_BYTES = QN * BK * 4;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;
constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int CL = 4;        // CTAs per cluster

struct GemmMcArgs {
  float* C;
  long long ldc;
  int M, N, K;
  int epi;
  const float* bnorm;
  float* row_min;
  int* row_arg;
  int rank;
  PclStatus* status;
};

// 64 rows of B into the same shared-memory offset of every CTA in `mask`; the bytes each CTA
// receives are counted on the barrier at `leader_bar`'s offset in the leader of ITS pair
__device__ __forceinline__ void tma_load_2d_pair_mc(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar,
                                                    int x, int y, uint16_t mask) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".multicast::cluster [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "h"(mask)
      : "memory");
}

// one arrival on the barrier at `bar`'s offset in every CTA of `mask`, once the MMAs issued so far
// by this thread have finished
__device__ __forceinline__ void umma_commit_mc(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}

__device__ __forceinline__ void abort_cluster(volatile int* abort_flag) {
  const uint32_t addr = smem_u32((const void*)abort_flag);
  for (uint32_t r = 0; r < (uint32_t)CL; ++r)
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(addr, r)), "r"(1) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tf32_2sm_mc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, GemmMcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (a.N + TN - 1) / TN;
  const int m_tiles = (a.M + TM - 1) / TM;
  const int m_pairs = (m_tiles + 1) / 2;
  const int kb_count = (a.K + BK - 1) / BK;

  const uint32_t crank = cluster_ctarank();   // 0..3
  const uint32_t me = crank & 1u;             // position in the pair (0 = leader)
  const uint32_t pj = crank >> 1;             // which pair of the cluster
  const uint32_t leader = crank & ~1u;
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + STAGES * A_BYTES;
  uint8_t* sE = base + STAGES * (A_BYTES + B_BYTES);
  uint64_t* bars = (uint64_t*)(sE + EPI_BYTES);
  uint64_t* full = bars;                 // STAGES, used in the pair leaders
  uint64_t* empty = bars + STAGES;       // STAGES, one set per CTA, two arrivals (one per pair)
  uint64_t* tfull = bars + 2 * STAGES;   // 2, one set per CTA
  uint64_t* tempty = tfull + 2;          // 2, used in the pair leaders
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 2); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull + b, 1); mbar_init(tempty + b, 2 * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)), "r"(2 * TN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the other CTAs' barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int cluster = (int)blockIdx.x / CL;
  const int nclusters = (int)gridDim.x / CL;
  // Work items of a cluster: with a stored C every (pair of row blocks, column tile), row-block
  // major; with the arg-min epilogue a pair of row blocks whose CTA pairs walk all column tiles.
  const bool flat = (a.epi == 0);
  const long long items = flat ? (long long)m_pairs * n_tiles : (long long)m_pairs;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint16_t bmask = (uint16_t)((1u << me) | (1u << (2u + me)));
      for (long long item = cluster; item < items && ok; item += nclusters) {
        const int mt = 2 * (int)(flat ? item / n_tiles : item) + (int)pj;
        const int nt0 = flat ? (int)(item % n_tiles) : 0;
        const int nt1 = flat ? nt0 + 1 : n_tiles;
        for (int nt = nt0; nt < nt1 && ok; ++nt) {
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(empty + stage, phase ^ 1, abort_flag)) {
              report(a.status, a.rank, 41, kb, stage);
              abort_cluster(abort_flag);
              ok = false;
              break;
            }
            if (me == 0) mbar_expect_tx(full + stage, 2 * (A_BYTES + B_BYTES));
            const uint32_t lbar = map_to_cta(smem_u32(full + stage), leader);
            tma_load_2d_pair(map_to_cta(smem_u32(sA + stage * A_BYTES), crank), &tmA, lbar, kb * BK,
                             mt * TM + (int)me * HM);
            tma_load_2d_pair_mc(map_to_cta(smem_u32(sB + stage * B_BYTES + (int)pj * Q_BYTES), crank), &tmB,
                                lbar, kb * BK, nt * TN + (int)me * HN + (int)pj * QN, bmask);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
      if (!ok) {
        for (int s = 0; s < 2048; ++s) __nanosleep(1000);  // let copies in flight land
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && me == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) |
                             ((uint32_t)(TM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      for (long long item = cluster; item < items && ok; item += nclusters) {
        const int nt0 = flat ? (int)(item % n_tiles) : 0;
        const int nt1 = flat ? nt0 + 1 : n_tiles;
        for (int nt = nt0; nt < nt1 && ok; ++nt) {
          if (!mbar_wait(tempty + acc, acc_phase[acc] ^ 1, abort_flag)) {
            report(a.status, a.rank, 42, acc, 0);
            abort_cluster(abort_flag);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t d = tmem_base + (uint32_t)(acc * TN);
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(full + stage, phase, abort_flag)) {
              report(a.status, a.rank, 43, kb, stage);
              abort_cluster(abort_flag);
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = make_desc_sw128(smem_u32(sA + stage * A_BYTES));
            const uint64_t db = make_desc_sw128(smem_u32(sB + stage * B_BYTES));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_tf32_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
            // this pair is done with the stage: tell the producers of all four CTAs
            umma_commit_mc(smem_u32(empty + stage), (uint16_t)0xF);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit_pair(map_to_cta(smem_u32(tfull + acc), leader));
          umma_commit_pair(map_to_cta(smem_u32(tfull + acc), leader + 1));
          acc_phase[acc] ^= 1;
          acc ^= 1;
        }
      }
    }
  } else {
    const int sub = warp & 3;                 // tensor-memory sub-partition of this warp
    const int half = (warp - 2) >> 2;         // which 128 of the tile's 256 columns
    constexpr int HC = TN / 2;                // columns per epilogue warp
    float* stg = reinterpret_cast<float*>(sE + (warp - 2) * 4096);
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(tempty), leader);
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    const bool vec_ok = ((a.ldc & 3) == 0) && ((((uintptr_t)a.C) & 15) == 0);
    for (long long item = cluster; item < items && ok; item += nclusters) {
      const int mt = 2 * (int)(flat ? item / n_tiles : item) + (int)pj;
      const int nt0 = flat ? (int)(item % n_tiles) : 0;
      const int nt1 = flat ? nt0 + 1 : n_tiles;
      const int row_base = mt * TM + (int)me * HM + sub * 32;   // first row of this warp's 32
      const int row = row_base + lane;
      float best = 3.402823466e38f;
      int best_n = 0;
      for (int nt = nt0; nt < nt1 && ok; ++nt) {
        if (!mbar_wait(tfull + acc, acc_phase[acc], abort_flag)) {
          if (lane == 0) {
            report(a.status, a.rank, 44, acc, 0);
            abort_cluster(abort_flag);
          }
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t0 = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(acc * TN);
        if (a.epi == 1) {   // |b_n|^2 of this tile's columns, +inf beyond N
          __syncwarp();
          for (int q = lane; q < HC; q += 32) {
            const int n = nt * TN + half * HC + q;
            stg[q] = n < a.N ? __ldg(a.bnorm + n) : 3.402823466e38f;
          }
          __syncwarp();
        }
        uint32_t rv[2][32];
        tmem_ld32_issue(t0 + (uint32_t)(half * HC), rv[0]);
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t* cur = rv[c & 1];
          tmem_ld_wait(cur);
          if (c + 1 < HC / 32) {
            tmem_ld32_issue(t0 + (uint32_t)(half * HC + (c + 1) * 32), rv[(c + 1) & 1]);
          } else {
            // the last chunk is in registers: hand the accumulator buffer back before its stores
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + (uint32_t)(acc * 8));
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(cur[j]);
          const int n0 = nt * TN + half * HC + c * 32;
          if (n0 >= a.N || row_base >= a.M) continue;
          if (a.epi == 0) {
            if (vec_ok) {
              // lane r writes accumulator row r into the staging buffer with the 128-byte swizzle;
              // one bulk tensor store moves the 32 x 32 box to C (clipped at the edges of C)
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              __syncwarp();
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(stg + lane * 32 + ((q ^ (lane & 7)) << 2)) =
                    make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) tma_store_2d(&tmC, smem_u32(stg), n0, row_base);
            } else if (row < a.M) {
              float* dst = a.C + (long long)row * a.ldc + n0;
              for (int j = 0; j < 32; ++j)
                if (n0 + j < a.N) dst[j] = v[j];
            }
          } else {
            float d[32];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 b = *reinterpret_cast<const float4*>(stg + c * 32 + 4 * q);
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
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
      if (ok && a.epi == 1 && row < a.M) {   // one result per column half; the caller merges the two
        a.row_min[(long long)half * a.M + row] = best;
        a.row_arg[(long long)half * a.M + row] = best_n;
      }
    }
    // the staging buffer must stay intact until the copy engine has read it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }

  // nobody leaves while another CTA may still write this CTA's shared memory or signal its barriers
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TN));
  }
}

}  // namespace

// C = A B^T (epi 0) or the row-wise arg-min of bnorm[n] - 2 A B^T (epi 1; row_min / row_arg hold
// 2 x M entries like pcl_gemm_tf32_2sm).  A, B and C must be memory of the launching device.
// Returns cudaErrorNotSupported when the device cannot co-schedule a cluster of four such CTAs.
PCL_API int pcl_gemm_tf32_2sm_mc(const float* A, const float* B, float* C, int M, int N, int K,
                                 long long ldc, int epi, const float* bnorm, float* row_min, int* row_arg,
                                 PclStatus* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 3) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return (int)cudaErrorInvalidValue;
  if (epi == 0 && C == nullptr) return (int)cudaErrorInvalidValue;
  if (epi == 1 && (bnorm == nullptr || row_min == nullptr || row_arg == nullptr))
    return (int)cudaErrorInvalidValue;
  // the operands must belong to the device that runs the kernel
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  const void* ptrs[3] = {A, B, C};
  for (const void* p : ptrs) {
    if (p == nullptr) continue;
    cudaPointerAttributes at;
    e = cudaPointerGetAttributes(&at, p);
    if (e != cudaSuccess) return (int)e;
    if (at.type != cudaMemoryTypeDevice || at.device != dev) return (int)cudaErrorInvalidDevice;
  }
  CUtensorMap tmA, tmB, tmC;
  int rc = make_map2(&tmA, A, M, K, HM, BK);
  if (rc) return rc;
  rc = make_map2(&tmB, B, N, K, QN, BK);
  if (rc) return rc;
  const bool c_ok = (epi == 0) && ((ldc & 3) == 0) && ((((uintptr_t)C) & 15) == 0);
  rc = c_ok ? make_map_c(&tmC, C, M, N, ldc) : make_map2(&tmC, A, M, K, HM, BK);
  if (rc) return rc;
  GemmMcArgs a;
  a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.epi = epi;
  a.bnorm = bnorm; a.row_min = row_min; a.row_arg = row_arg;
  a.rank = 0; a.status = status;

  e = cudaFuncSetAttribute(gemm_tf32_2sm_mc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // the grid is persistent: as many clusters as the device can hold at once
  static int max_clusters = -1;
  if (max_clusters < 0) {
    cfg.gridDim = dim3(CL, 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tf32_2sm_mc_kernel, &cfg);
    if (e != cudaSuccess) return (int)e;
    max_clusters = n;
  }
  int clusters = max_clusters;
  if (num_sms > 0 && num_sms / CL < clusters) clusters = num_sms / CL;
  if (clusters < 1) return (int)cudaErrorNotSupported;
  const int m_pairs = ((M + TM - 1) / TM + 1) / 2;
  const long long n_items = (epi == 0) ? (long long)m_pairs * ((N + TN - 1) / TN) : (long long)m_pairs;
  if (clusters > n_items) clusters = (int)n_items;
  cfg.gridDim = dim3((unsigned)(CL * clusters), 1, 1);
  e = cudaLaunchKernelEx(&cfg, gemm_tf32_2sm_mc_kernel, tmA, tmB, tmC, a);
  if (e != cudaSuccess) return (int)e;
  return pcl_last_error();
}
