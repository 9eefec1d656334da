// Device-side SSP clock (stale-synchronous-parallel bounded staleness).
//
// Reference behaviour being replaced: iter_commit() does a TCP round trip to a
// dedicated server thread that counts commits per clock slot and advances
// `server_clock` (include/ps.hpp:343-355, include/server.hpp:114-167); readers
// poll `server_clock` over TCP until stale_cache + limit_s >= clock
// (ps.hpp:447-457).  Here every rank owns an array clocks[world] of 64-bit
// words in memory that its peers can address.  A commit is one release store of
// the rank's new clock into slot [rank] of every peer's array; the staleness
// test is min(clocks) >= clock - s evaluated by a bounded spin on local memory.
// A rank that has finished all its iterations commits PCL_CLOCK_DEPARTED so
// that nobody waits for it again (the reference decrements worker_sz instead,
// ps.hpp:352-354).
#include "common.cuh"

namespace {

__global__ void ssp_commit_kernel(long long* const* clock_ptrs, int world, int rank,
                                  long long value, const PclStatus* status) {
  // a rank whose wait ran out (or that met a bad id) this round does not announce progress
  if (pcl_status_code(status) != 0) return;
  int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();  // order this rank's earlier pushes before the clock
    pcl_st_release_sys(clock_ptrs[r] + rank, value);
  }
}

__global__ void ssp_wait_kernel(const long long* clocks, int world, long long target,
                                unsigned long long timeout_ns, PclStatus* st, int rank) {
  if (threadIdx.x == 0 && blockIdx.x == 0)
    pcl_wait_min_clock(clocks, world, target, timeout_ns, st, rank, 2);
}

}  // namespace

PCL_API int pcl_ssp_commit(long long* const* clock_ptrs, int world, int rank, long long value,
                           const PclStatus* status, cudaStream_t stream) {
  if (world > 1024) return (int)cudaErrorInvalidValue;
  ssp_commit_kernel<<<1, ((world + 31) / 32) * 32, 0, stream>>>(clock_ptrs, world, rank, value,
                                                                status);
  return pcl_last_error();
}

PCL_API int pcl_ssp_wait(const long long* clocks, int world, long long target,
                         unsigned long long timeout_ns, PclStatus* status, int rank,
                         cudaStream_t stream) {
  ssp_wait_kernel<<<1, 32, 0, stream>>>(clocks, world, target, timeout_ns, status, rank);
  return pcl_last_error();
}
