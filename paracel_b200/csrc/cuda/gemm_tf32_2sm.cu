// C[M x N] = A[M x K] * B[N x K]^T, fp32 storage, tcgen05.mma kind::tf32 with
// cta_group::2: two CTAs on neighbouring SMs (a cluster of two) work on one
// 256 x 256 output tile.  Each CTA stages only ITS half of the operands per K
// step (128 rows of A, 128 rows of B: 32 KB instead of the 64 KB a lone CTA
// would need for the same number of flops), the tensor cores of both SMs read
// both halves, and each CTA keeps its 128 x 256 half of the accumulator in its
// own tensor memory.  Shared-memory traffic per flop is half of the
// one-CTA kernel in gemm_tf32.cu, which is bound by exactly that traffic.
//
// Same contract as pcl_gemm_tf32 (store or k-means arg-min epilogue, fused
// all-gather of a range-sharded B through a local staging buffer).  Reference
// call sites that this serves: the centre-distance loop of
// alg/clustering/kmeans/kmeans.hpp:113-133 and the all-pairs products of
// alg/recommendation/similarity_dense/sim_dense.hpp:84-101.
//
// Two item forms, chosen by the launcher:
//   256 x 256 items, two accumulators that alternate (the epilogue of one tile runs under the
//     main loop of the next), six 32 KB operand stages per CTA;
//   256 x 512 items, two accumulators fed from the same A stage (24 KB instead of 32 KB of
//     operands per 256 x 256 x 32 block of MACs), four 48 KB stages; the epilogue of an item
//     overlaps only with the operand prefetch of the next, so this form pays for long K only.
//
// Roles in each CTA (320 threads):
//   warp 0      TMA producer for this CTA's operand halves; the transfers of both
//               CTAs complete on the LEADER's "full" barrier (cta_group::2 form of
//               cp.async.bulk.tensor, no multicast)
//   warp 1      tensor-memory allocation (both CTAs); in the leader one lane issues
//               the M256 N256 K8 MMAs and commits to the barriers of both CTAs
//   warps 2-9   epilogue on the CTA's own accumulator half, two warps per tensor-memory
//               sub-partition (each takes 128 of the 256 columns): tcgen05.ld of the next
//               32 x 32 chunk is in flight while the current one is written, with the
//               128-byte swizzle, into the warp's staging buffer and handed to a bulk tensor
//               store (cp.async.bulk.tensor shared -> global, local memory; stores have no
//               multicast form), which clips at the edges of C; or the arg-min.  The
//               accumulator is released as soon as its last chunk is in registers.
// Measured and not kept for the epilogue: two staging buffers per warp with five operand stages
// (slower on every shape), coalesced 128-bit global stores out of the staging buffer (8 % slower),
// 256-bit stores straight from the registers (17 % slower), L2 evict-first / evict-last hints on
// the C stores and the B loads (within 2 %), a start-up stagger between the pairs (no change).
// Measured and not kept for the main loop: stages of 16 elements of K (64-byte rows, 64-byte
// swizzle, twelve or eight stages instead of six or four, so that a larger share of the operand
// memory is in flight): numerically identical, but 428 against 583 TFLOP/s at 65536 x 16384 x 512 and
// 555 against 701 at 8192^3; the copy engine and L2 do worse on half-line rows than the deeper ring gains.
// Every wait has a time limit; on expiry the status record is written, both
// CTAs of the pair are told to leave, tensor memory is freed and the kernel ends.
#include <cuda.h>

#include "common.cuh"
#include "gemm_sm100.cuh"

namespace {

using namespace pcl_sm100;

constexpr int TM = 256;      // tile rows per CTA pair
constexpr int TN = 256;      // columns per accumulator
constexpr int HM = 128;      // rows of A (and of the accumulator) per CTA
constexpr int HN = 128;      // rows of B staged per CTA and accumulator
constexpr int BK = 32;       // 32 fp32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;
constexpr int A_BYTES = HM * BK * 4;
constexpr int B_BYTES = HN * BK * 4;
constexpr int OPERAND_BYTES = 6 * (A_BYTES + B_BYTES);   // 192 KB of operand stages in either form
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;           // one 4 KB staging buffer per epilogue warp
constexpr int SMEM_BYTES = OPERAND_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int MAX_STAGES = 6;

struct Gemm2Args {
  float* C;
  long long ldc;
  int M, N, K;
  int epi;
  const float* bnorm;
  float* row_min;
  int* row_arg;
  const float* const* b_shards;
  float* b_stage;
  int* flags;          // one per 256-column tile
  int world, rank, rows_per_shard, epoch, gather_ctas;
  int group;           // row blocks per raster group (0: row-block major)
  PclStatus* status;
};

__device__ __forceinline__ int tile_at(int ord, int n_tiles, int first_local) {
  const int t = first_local + ord;
  return t >= n_tiles ? t - n_tiles : t;
}

// The order in which a pair walks the output.  A work item is a 256-row block `mt` with the
// column tiles of positions [ord0, ord1) of the rank's tile order (tile_at): NH of them with a
// stored C, all of them with the arg-min epilogue (the caller then steps through them NH at a time).
template <int NH>
struct Schedule {
  bool flat;
  int n_tiles, m_tiles, n_first, ipr1, ipr2, group;
  long long first_items, items;

  __device__ Schedule(const Gemm2Args& a, int n_tiles_, int m_tiles_) {
    flat = (a.epi == 0);
    n_tiles = n_tiles_;
    m_tiles = m_tiles_;
    // With a fused gather the stored form has two phases: every row block against this rank's own
    // column tiles first (their staging is a local copy), then against the tiles of the peers.
    n_first = n_tiles;
    if (a.gather_ctas > 0) {
      const int own_rows = max(0, min(a.rows_per_shard, a.N - a.rank * a.rows_per_shard));
      n_first = max(1, min(n_tiles, own_rows / TN));
    }
    ipr1 = (n_first + NH - 1) / NH;
    ipr2 = (n_tiles - n_first + NH - 1) / NH;
    group = (flat && a.gather_ctas == 0) ? a.group : 0;
    first_items = (long long)m_tiles * ipr1;
    items = flat ? (long long)m_tiles * (ipr1 + ipr2) : (long long)m_tiles;
  }

  __device__ void decode(long long item, int& mt, int& ord0, int& ord1) const {
    if (!flat) {
      mt = (int)item; ord0 = 0; ord1 = n_tiles;
    } else if (group > 0) {
      // groups of `group` row blocks, column-tile major inside a group: the pairs that run together
      // then touch `group` row blocks of A and about (pairs / group) tiles of B instead of one
      // row block and every tile of B
      const long long per = (long long)group * ipr1;
      const long long g = item / per;
      const int r = (int)(item - g * per);
      const int rows = (int)min((long long)group, (long long)m_tiles - g * group);
      mt = (int)(g * group) + r % rows;
      ord0 = (r / rows) * NH; ord1 = min(ord0 + NH, n_tiles);
    } else if (item < first_items) {
      mt = (int)(item / ipr1);
      ord0 = (int)(item % ipr1) * NH; ord1 = min(ord0 + NH, n_first);
    } else {
      const long long rem = item - first_items;
      mt = (int)(rem / ipr2);
      ord0 = n_first + (int)(rem % ipr2) * NH; ord1 = min(ord0 + NH, n_tiles);
    }
  }
};

// raise the abort flag of both CTAs of the pair
__device__ __forceinline__ void abort_pair(volatile int* abort_flag, uint32_t peer) {
  *abort_flag = 1;
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(smem_u32((const void*)abort_flag), peer)),
               "r"(1)
               : "memory");
}

// NH = 1: one 256 x 256 accumulator per item, two of them alternate (the epilogue of a tile runs
//         under the main loop of the next), six 32 KB operand stages per CTA.
// NH = 2: a 256 x 512 item, both accumulators fed from the same A stage; four 48 KB stages.
template <int NH>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tf32_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, Gemm2Args a) {
  constexpr int STAGES = (NH == 2) ? 4 : 6;
  constexpr int STAGE_BYTES = A_BYTES + NH * B_BYTES;
  static_assert(STAGES * STAGE_BYTES == OPERAND_BYTES, "operand stages fill the same 192 KB");
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (a.N + TN - 1) / TN;
  const int m_tiles = (a.M + TM - 1) / TM;
  const int kb_count = (a.K + BK - 1) / BK;
  int first_local = 0;
  if (a.world > 1) first_local = (int)(((long long)a.rank * a.rows_per_shard) / TN) % n_tiles;


  // ------------------------------------------------- gather CTAs (whole clusters)
  // One thread per gather CTA drives the copy engine of its SM: contiguous pieces of a peer's
  // shard (up to 32 KB) are fetched into shared memory with cp.async.bulk (a plain bulk load, no
  // multicast; the source is the peer's memory over NVLink), and each piece that has landed goes
  // on to the local staging buffer with a bulk store.  GBUF pieces are in flight per CTA, which
  // is what the NVLink latency needs: with 128-bit loads issued by the CTA's threads a CTA moved
  // about 20 GB/s and sixteen CTAs had to be taken from the tensor cores.
  if ((int)blockIdx.x < a.gather_ctas) {
    constexpr int GBUF = 6;
    constexpr uint32_t GCH = 32768;
    uint8_t* gbase = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* gbar = (uint64_t*)(gbase + GBUF * GCH);
    __shared__ int g_abort;
    if (threadIdx.x == 0) {
      for (int i = 0; i < GBUF; ++i) mbar_init(gbar + i, 1);
      g_abort = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const long long row_bytes = (long long)a.K * 4;
    // the pieces of this CTA's tiles form one sequence; piece q uses buffer q % GBUF
    struct Piece { const uint8_t* src; uint8_t* dst; uint32_t bytes; int tile_end; };
    auto piece_at = [&](int ord, long long off_in_tile, Piece& pc) -> bool {
      // tile `ord` of this CTA's list; off_in_tile counts bytes from the tile's first row
      const int nt = tile_at(ord, n_tiles, first_local);
      const long long r0 = (long long)nt * TN;
      const long long r1 = min((long long)a.N, r0 + TN);
      const long long tile_bytes = (r1 - r0) * row_bytes;
      if (off_in_tile >= tile_bytes) return false;
      const long long row = r0 + off_in_tile / row_bytes;
      const int owner = (int)min(row / a.rows_per_shard, (long long)a.world - 1);
      const long long owner_end_row = min(r1, (long long)(owner + 1) * a.rows_per_shard +
                                                  (owner == a.world - 1 ? (long long)a.N : 0));
      const long long seg_end = (owner_end_row - r0) * row_bytes;     // end of this owner's part of the tile
      long long n = seg_end - off_in_tile;
      if (n > GCH) n = GCH;
      pc.src = reinterpret_cast<const uint8_t*>(a.b_shards[owner]) +
               (row - (long long)owner * a.rows_per_shard) * row_bytes + off_in_tile % row_bytes;
      pc.dst = reinterpret_cast<uint8_t*>(a.b_stage) + r0 * row_bytes + off_in_tile;
      pc.bytes = (uint32_t)n;
      pc.tile_end = (off_in_tile + n >= tile_bytes) ? nt : -1;
      return true;
    };
    // two cursors over the same piece sequence: `ld` issues loads GBUF pieces ahead of `st`
    int ld_ord = blockIdx.x, st_ord = blockIdx.x;
    long long ld_off = 0, st_off = 0;
    long long issued = 0, stored = 0;
    bool ok = true;
    auto issue_load = [&]() {
      Piece pc;
      while (ld_ord < n_tiles && !piece_at(ld_ord, ld_off, pc)) { ld_ord += a.gather_ctas; ld_off = 0; }
      if (ld_ord >= n_tiles) return false;
      const int bidx = (int)(issued % GBUF);
      mbar_expect_tx(gbar + bidx, pc.bytes);
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          ::"r"(smem_u32(gbase + bidx * GCH)), "l"(pc.src), "r"(pc.bytes), "r"(smem_u32(gbar + bidx))
          : "memory");
      ld_off += pc.bytes;
      ++issued;
      return true;
    };
    for (int i = 0; i < GBUF; ++i)
      if (!issue_load()) break;
    while (stored < issued && ok) {
      Piece pc;
      while (!piece_at(st_ord, st_off, pc)) { st_ord += a.gather_ctas; st_off = 0; }
      const int bidx = (int)(stored % GBUF);
      if (!mbar_wait(gbar + bidx, (uint32_t)((stored / GBUF) & 1), &g_abort)) {
        report(a.status, a.rank, 35, stored, bidx);
        ok = false;
        break;
      }
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(pc.dst),
                   "r"(smem_u32(gbase + bidx * GCH)), "r"(pc.bytes)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      st_off += pc.bytes;
      ++stored;
      if (pc.tile_end >= 0) {
        // the tile is complete once every store so far has been written
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        __threadfence();
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(a.flags + pc.tile_end), "r"(a.epoch) : "memory");
      } else {
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the buffer may be refilled
      }
      issue_load();
    }
    if (!ok) {
      // give the loads that are still in flight time to land before the shared memory goes away
      for (int s_ = 0; s_ < 2048; ++s_) __nanosleep(1000);
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    return;
  }


  // ------------------------------------------------------------------ MMA pairs
  const uint32_t me = cluster_ctarank();   // 0 = leader
  const uint32_t peer = me ^ 1u;
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sOp = base;                   // stage s: A at s * STAGE_BYTES, B of accumulator h behind it
  uint8_t* sE = base + OPERAND_BYTES;
  uint64_t* bars = (uint64_t*)(sE + EPI_BYTES);
  uint64_t* full = bars;                     // STAGES, used in the leader
  uint64_t* empty = bars + MAX_STAGES;       // STAGES, one set per CTA
  uint64_t* tfull = bars + 2 * MAX_STAGES;   // 2, one set per CTA
  uint64_t* tempty = tfull + 2;              // 2, used in the leader (one arrival per epilogue warp of the pair)
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
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
  cluster_sync_all();   // the peer's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int pair = ((int)blockIdx.x - a.gather_ctas) >> 1;
  const int npair = ((int)gridDim.x - a.gather_ctas) >> 1;
  const Schedule<NH> sch(a, n_tiles, m_tiles);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long item = pair; item < sch.items && ok; item += npair) {
        int mt, ord0, ord1;
        sch.decode(item, mt, ord0, ord1);
        for (int ord = ord0; ord < ord1 && ok; ord += NH) {
          int nts[NH];
          int nvalid = 0;
#pragma unroll
          for (int h = 0; h < NH; ++h) {
            nts[h] = (ord + h < ord1) ? tile_at(ord + h, n_tiles, first_local) : -1;
            nvalid += nts[h] >= 0;
          }
          if (a.gather_ctas > 0) {
#pragma unroll
            for (int h = 0; h < NH; ++h) {
              if (nts[h] < 0 || !ok) continue;
              int seen = 0;
              const unsigned long long t0 = pcl_globaltimer();
              for (unsigned it = 0;; ++it) {
                seen = pcl_ld_acquire_sys_i32(a.flags + nts[h]);
                if (seen == a.epoch || *abort_flag) break;
                if ((it & 15) == 15 && pcl_globaltimer() - t0 > WAIT_NS) break;
                __nanosleep(128);
              }
              if (seen != a.epoch) {
                report(a.status, a.rank, 30, a.epoch, seen);
                abort_pair(abort_flag, peer);
                ok = false;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(empty + stage, phase ^ 1, abort_flag)) {
              report(a.status, a.rank, 31, kb, stage);
              abort_pair(abort_flag, peer);
              ok = false;
              break;
            }
            if (me == 0) mbar_expect_tx(full + stage, 2u * (uint32_t)(A_BYTES + nvalid * B_BYTES));
            const uint32_t lbar = map_to_cta(smem_u32(full + stage), 0);
            uint8_t* st = sOp + stage * STAGE_BYTES;
            tma_load_2d_pair(map_to_cta(smem_u32(st), me), &tmA, lbar, kb * BK, mt * TM + (int)me * HM);
#pragma unroll
            for (int h = 0; h < NH; ++h)
              if (nts[h] >= 0)
                tma_load_2d_pair(map_to_cta(smem_u32(st + A_BYTES + h * B_BYTES), me), &tmB, lbar, kb * BK,
                                 nts[h] * TN + (int)me * HN);
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
      for (long long item = pair; item < sch.items && ok; item += npair) {
        int mt, ord0, ord1;
        sch.decode(item, mt, ord0, ord1);
        for (int ord = ord0; ord < ord1 && ok; ord += NH) {
          for (int kb = 0; kb < kb_count && ok; ++kb) {
            if (!mbar_wait(full + stage, phase, abort_flag)) {
              report(a.status, a.rank, 33, kb, stage);
              abort_pair(abort_flag, peer);
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint8_t* st = sOp + stage * STAGE_BYTES;
            const uint64_t da = make_desc_sw128(smem_u32(st));
#pragma unroll
            for (int h = 0; h < NH; ++h) {
              if (ord + h >= ord1) continue;
              const int slot = (NH == 2) ? h : acc;
              if (kb == 0) {   // the epilogue has drained what this accumulator held before
                if (!mbar_wait(tempty + slot, acc_phase[slot] ^ 1, abort_flag)) {
                  report(a.status, a.rank, 32, slot, 0);
                  abort_pair(abort_flag, peer);
                  ok = false;
                  break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              }
              const uint32_t d = tmem_base + (uint32_t)(slot * TN);
              const uint64_t db = make_desc_sw128(smem_u32(st + A_BYTES + h * B_BYTES));
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                umma_tf32_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                               (kb > 0 || k > 0) ? 1u : 0u);
              if (kb == kb_count - 1) {   // this accumulator is complete once these MMAs are
                umma_commit_pair(map_to_cta(smem_u32(tfull + slot), 0));
                umma_commit_pair(map_to_cta(smem_u32(tfull + slot), 1));
                acc_phase[slot] ^= 1;
              }
            }
            if (!ok) break;
            // free this stage in both CTAs
            umma_commit_pair(map_to_cta(smem_u32(empty + stage), 0));
            umma_commit_pair(map_to_cta(smem_u32(empty + stage), 1));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (NH == 1) acc ^= 1;
        }
      }
    }
  } else {
    const int sub = warp & 3;                 // tensor-memory sub-partition of this warp
    const int half = (warp - 2) >> 2;         // which 128 of the accumulator's 256 columns
    constexpr int HC = TN / 2;                // columns per epilogue warp
    float* stg = reinterpret_cast<float*>(sE + (warp - 2) * 4096);
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(tempty), 0);
    const bool vec_ok = ((a.ldc & 3) == 0) && ((((uintptr_t)a.C) & 15) == 0);
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    for (long long item = pair; item < sch.items && ok; item += npair) {
      int mt, ord0, ord1;
      sch.decode(item, mt, ord0, ord1);
      const int row_base = mt * TM + (int)me * HM + sub * 32;   // first row of this warp's 32
      const int row = row_base + lane;
      float best = 3.402823466e38f;
      int best_n = 0;
      for (int ord = ord0; ord < ord1 && ok; ord += NH) {
#pragma unroll 1
        for (int h = 0; h < NH; ++h) {
          if (ord + h >= ord1 || !ok) continue;
          const int nt = tile_at(ord + h, n_tiles, first_local);
          const int slot = (NH == 2) ? h : acc;
          if (!mbar_wait(tfull + slot, acc_phase[slot], abort_flag)) {
            if (lane == 0) {
              report(a.status, a.rank, 34, slot, 0);
              abort_pair(abort_flag, peer);
            }
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t t0 = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(slot * TN);
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
              // the last chunk is in registers: hand the accumulator back before its stores
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(tempty_leader0 + (uint32_t)(slot * 8));
            }
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(cur[j]);
            const int n0 = nt * TN + half * HC + c * 32;
            if (n0 >= a.N) continue;
            if (a.epi == 0) {
              if (vec_ok) {
                // lane r writes accumulator row r into the staging buffer with the 128-byte swizzle
                // (16-byte chunk q of row r sits at chunk q ^ (r & 7)); one bulk tensor store then
                // moves the 32 x 32 box to C.  The buffer is free again once the store that read it
                // last has finished reading.
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
              // dist[j] = |b_n|^2 - 2 a.b_n; the minimum first (one FMNMX per column), the column
              // index only when this chunk improves the running best, which becomes rare quickly
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
          acc_phase[slot] ^= 1;
        }
        if (NH == 1) acc ^= 1;
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

  // nobody leaves while the peer may still read this CTA's shared memory or signal its barriers
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TN));
  }
}

template <int NH>
int launch_2sm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, Gemm2Args& a,
               int num_sms, cudaStream_t stream) {
  auto kern = gemm_tf32_2sm_kernel<NH>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // every cluster of the grid must be resident at once: MMA pairs wait for the gather CTAs
  static int max_clusters = -1;
  if (max_clusters < 0) {
    cfg.gridDim = dim3(2, 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return (int)e;
    max_clusters = n;
  }
  int clusters = max_clusters;
  if (num_sms > 0 && num_sms / 2 < clusters) clusters = num_sms / 2;
  if (clusters < 1 + a.gather_ctas / 2) return (int)cudaErrorNotSupported;
  const int m_tiles = (a.M + TM - 1) / TM;
  const int n_tiles = (a.N + TN - 1) / TN;
  int mma_pairs = clusters - a.gather_ctas / 2;
  // an upper bound of the number of work items (the two-phase order of the fused gather can split
  // a row block's tiles into one more item than ceil(n_tiles / NH))
  const long long n_items = (a.epi == 0) ? (long long)m_tiles * ((n_tiles + NH - 1) / NH + 1) : (long long)m_tiles;
  if (mma_pairs > n_items) mma_pairs = (int)n_items;
  cfg.gridDim = dim3((unsigned)(a.gather_ctas + 2 * mma_pairs), 1, 1);
  e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, a);
  if (e != cudaSuccess) return (int)e;
  return pcl_last_error();
}

}  // namespace

// Same arguments as pcl_gemm_tf32, except that `flags` holds one int per 256-column tile,
// `gather_ctas` is rounded up to an even number, and with epi 1 row_min / row_arg hold 2 x M
// entries: [0..M) is the result over columns n with (n mod 256) < 128, [M..2M) over the others
// (the two epilogue warps of a row work on separate column halves; the caller takes the smaller).
// `wide`: 1 = 256 x 512 items (two accumulators fed from one A stage), 0 = 256 x 256 items with
// alternating accumulators, -1 = chosen here (wide for K >= 1024 with at least two column tiles).
// Returns cudaErrorNotSupported when the device cannot co-schedule a single pair of CTAs with
// this much shared memory.
PCL_API int pcl_gemm_tf32_2sm(const float* A, float* b_stage, float* C, int M, int N, int K,
                              long long ldc, int epi, const float* bnorm, float* row_min, int* row_arg,
                              const float* const* b_shards, int* flags, int world, int rank,
                              int rows_per_shard, int epoch, int gather_ctas, PclStatus* status,
                              int num_sms, int wide, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 3) || ((uintptr_t)A & 15) || ((uintptr_t)b_stage & 15)) return (int)cudaErrorInvalidValue;
  if (epi == 0 && C == nullptr) return (int)cudaErrorInvalidValue;
  if (epi == 1 && (bnorm == nullptr || row_min == nullptr || row_arg == nullptr))
    return (int)cudaErrorInvalidValue;
  CUtensorMap tmA, tmB, tmC;
  int rc = make_map2(&tmA, A, M, K, HM, BK);
  if (rc) return rc;
  rc = make_map2(&tmB, b_stage, N, K, HN, BK);
  if (rc) return rc;
  // bulk tensor stores need a 16-byte aligned base and row stride; otherwise (and for the arg-min
  // epilogue) the map is a stand-in over A that the kernel never uses
  const bool c_ok = (epi == 0) && ((ldc & 3) == 0) && ((((uintptr_t)C) & 15) == 0);
  rc = c_ok ? make_map_c(&tmC, C, M, N, ldc) : make_map2(&tmC, A, M, K, HM, BK);
  if (rc) return rc;
  Gemm2Args a;
  a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.epi = epi;
  a.bnorm = bnorm; a.row_min = row_min; a.row_arg = row_arg;
  a.b_shards = b_shards; a.b_stage = b_stage; a.flags = flags;
  a.world = world; a.rank = rank; a.rows_per_shard = rows_per_shard > 0 ? rows_per_shard : N;
  a.epoch = epoch; a.status = status;
  const bool fused = (world > 1 && b_shards != nullptr);
  a.gather_ctas = fused ? (gather_ctas > 0 ? ((gather_ctas + 1) & ~1) : 16) : 0;
  if (fused && flags == nullptr) return (int)cudaErrorInvalidValue;
  // Measured on 65536 x 16384 and 8192 x 8192 outputs, the forms interleaved in one process:
  // K = 512: 566 TFLOP/s with 256 x 256 items, 509 with 256 x 512; K = 1024: 406 against 594;
  // K = 8192: 550 against 619, and 667 with raster groups.  Groups of eight row blocks pay once B
  // is larger than the L2 cache (K = 8192: B is 268 MB) and cost up to a tenth below that.
  a.group = ((long long)N * K * 4 >= (100ll << 20)) ? 8 : 0;
  const int n_tiles = (N + TN - 1) / TN;
  if (wide < 0) wide = (n_tiles >= 2 && K >= 1024) ? 1 : 0;
  return wide ? launch_2sm<2>(tmA, tmB, tmC, a, num_sms, stream)
              : launch_2sm<1>(tmA, tmB, tmC, a, num_sms, stream);
}
