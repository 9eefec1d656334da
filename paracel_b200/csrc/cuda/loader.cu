// Device side of the distributed load: placement of parsed (row, col, weight)
// triples on the rank grid and their exchange, written as an all-to-all whose
// dispatch is fused with the bucket computation.  Each rank runs
//   partition_count    histogram of destination ranks of its triples
//   partition_scatter  every triple is stored straight into the receive arrays of
//                      its destination rank (peer stores over NVLink), at the
//                      offset reserved for this source rank plus a running cursor
// with one host-side exchange of the count matrix in between.  Placement is the
// reference's  h(i, j) = (hash(i) % npx) * npy + hash(j) % npy  with the identity
// hash of 64-bit ids (include/load/scheduler.hpp:75-95, 115-155; the all-to-all
// it replaces: scheduler.hpp:157-170).
#include "common.cuh"

namespace {

__device__ __forceinline__ int dest_of(long long a, long long b, int npx, int npy) {
  return (int)((unsigned long long)a % (unsigned)npx) * npy + (int)((unsigned long long)b % (unsigned)npy);
}

__global__ void __launch_bounds__(256) partition_count_kernel(const long long* a, const long long* b,
                                                              long long n, int npx, int npy,
                                                              unsigned long long* counts) {
  extern __shared__ unsigned int hist[];
  const int world = npx * npy;
  for (int i = threadIdx.x; i < world; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    atomicAdd(&hist[dest_of(a[i], b[i], npx, npy)], 1u);
  __syncthreads();
  for (int i = threadIdx.x; i < world; i += blockDim.x)
    if (hist[i]) atomicAdd(&counts[i], (unsigned long long)hist[i]);
}

struct ScatterArgs {
  const long long* a;
  const long long* b;
  const float* w;
  long long n;
  int npx, npy;
  long long* const* recv;       // world base pointers; layout per rank: a[cap] | b[cap] | w[cap] (fp32)
  long long cap;                // capacity of each receive array (triples)
  const long long* base;        // [world] first slot of this source rank in destination d
  const long long* quota;       // [world] number of slots reserved there
  unsigned long long* cursor;   // [world] zero on entry
  PclStatus* status;
  int rank;
};

__global__ void __launch_bounds__(256) partition_scatter_kernel(ScatterArgs s) {
  const int lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n_round = (s.n + 31) / 32 * 32;   // whole warps stay in the loop together
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_round; i += stride) {
    const bool live = i < s.n;
    long long av = 0, bv = 0;
    float wv = 0.f;
    int d = -1;
    if (live) {
      av = s.a[i]; bv = s.b[i]; wv = s.w[i];
      d = dest_of(av, bv, s.npx, s.npy);
    }
    // one cursor update per (warp, destination)
    const unsigned peers = __match_any_sync(0xffffffffu, d);
    const int leader = __ffs(peers) - 1;
    const int my_slot = __popc(peers & ((1u << lane) - 1u));
    unsigned long long first = 0;
    if (live && lane == leader) first = atomicAdd(&s.cursor[d], (unsigned long long)__popc(peers));
    first = __shfl_sync(0xffffffffu, first, leader);
    if (!live) continue;
    const long long k = (long long)first + my_slot;
    if (k >= s.quota[d]) {   // more triples for d than were counted: refuse instead of overrunning
      if (atomicCAS(&s.status->code, 0, 2) == 0) {
        s.status->rank = s.rank; s.status->wait_id = 40; s.status->expected = s.quota[d]; s.status->seen = k;
      }
      continue;
    }
    const long long pos = s.base[d] + k;
    long long* r = s.recv[d];
    r[pos] = av;
    r[s.cap + pos] = bv;
    reinterpret_cast<float*>(r + 2 * s.cap)[pos] = wv;
  }
  __threadfence_system();
}

}  // namespace

// counts[world] (zeroed by the caller) += number of triples per destination rank.
PCL_API int pcl_partition_count(const long long* a, const long long* b, long long n, int npx, int npy,
                                unsigned long long* counts, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int world = npx * npy;
  if (world < 1 || world > 4096) return (int)cudaErrorInvalidValue;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  partition_count_kernel<<<(int)blocks, 256, world * sizeof(unsigned int), stream>>>(a, b, n, npx, npy, counts);
  return pcl_last_error();
}

// Stores every triple into the receive arrays of its destination (see ScatterArgs).
PCL_API int pcl_partition_scatter(const long long* a, const long long* b, const float* w, long long n,
                                  int npx, int npy, long long* const* recv, long long cap,
                                  const long long* base, const long long* quota,
                                  unsigned long long* cursor, PclStatus* status, int rank,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if (status == nullptr) return (int)cudaErrorInvalidValue;
  ScatterArgs s{a, b, w, n, npx, npy, recv, cap, base, quota, cursor, status, rank};
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  partition_scatter_kernel<<<(int)blocks, 256, 0, stream>>>(s);
  return pcl_last_error();
}
