// Shared device/host helpers for the sm_100a kernels of paracel_b200.
//
// Conventions used by every translation unit in this directory:
//   * every exported launcher is `extern "C" int pcl_<name>(..., cudaStream_t)`
//     and returns a cudaError_t value (0 = success) so that Python can call it
//     through ctypes without any C++ ABI;
//   * no exported launcher allocates memory unless its name says so;
//   * every device-side wait is bounded by a globaltimer deadline and reports
//     through a PclStatus word instead of trapping or spinning forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define PCL_API extern "C" __attribute__((visibility("default")))

// Status block written by kernels that can time out.  The host allocates it in
// device (or mapped) memory, zeroes it, and reads it back after the stream
// synchronises.  code: 0 ok, 1 wait timed out, 2 bad argument seen on device.
struct PclStatus {
  int code;
  int rank;
  int wait_id;
  int pad;
  long long expected;
  long long seen;
};

__device__ __forceinline__ unsigned long long pcl_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ long long pcl_ld_acquire_sys(const long long* p) {
  long long v;
  asm volatile("ld.acquire.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void pcl_st_release_sys(long long* p, long long v) {
  asm volatile("st.release.sys.global.s64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ int pcl_ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void pcl_st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 128-bit load that bypasses L1 (other SMs / other GPUs may have written it).
__device__ __forceinline__ float4 pcl_ldcg4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// 128-bit relaxed system-scope load: used for rows that live in a peer GPU.
__device__ __forceinline__ float4 pcl_ld_sys4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

// Vector reduction (no return value) of four floats; one L2 atomic per 16 B.
__device__ __forceinline__ void pcl_red_add4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ void pcl_red_add4_sys(float* p, float4 v) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ float pcl_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ double pcl_warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Bounded wait until min(clocks[0..world)) >= target.  Called by ONE thread.
// Returns true on success; on expiry fills *st (first writer wins) and returns
// false.  `clocks` is in this GPU's memory; peers store into it.
__device__ __forceinline__ bool pcl_wait_min_clock(const long long* clocks, int world,
                                                   long long target,
                                                   unsigned long long timeout_ns,
                                                   PclStatus* st, int rank, int wait_id) {
  unsigned long long t0 = pcl_globaltimer();
  long long seen = 0;
  for (;;) {
    long long m = 0x7fffffffffffffffLL;
    for (int r = 0; r < world; ++r) {
      long long c = pcl_ld_acquire_sys(clocks + r);
      m = c < m ? c : m;
    }
    seen = m;
    if (m >= target) return true;
    if (pcl_globaltimer() - t0 > timeout_ns) break;
    __nanosleep(200);
  }
  if (st != nullptr && atomicCAS(&st->code, 0, 1) == 0) {
    st->rank = rank;
    st->wait_id = wait_id;
    st->expected = target;
    st->seen = seen;
  }
  return false;
}

// A kernel met an id outside its table: record it (first writer wins) so that the host can raise
// after the stream synchronises.  `where` names the kernel (100 + n), `pos` the position of the id.
__device__ __forceinline__ void pcl_report_bad_id(PclStatus* st, int rank, int where, long long pos,
                                                  long long id) {
  if (st != nullptr && atomicCAS(&st->code, 0, 2) == 0) {
    st->rank = rank;
    st->wait_id = where;
    st->expected = pos;
    st->seen = id;
  }
}

// Current status code as the device sees it (0 when no status block was given).
__device__ __forceinline__ int pcl_status_code(const PclStatus* st) {
  return st != nullptr ? *reinterpret_cast<const volatile int*>(&st->code) : 0;
}

static inline int pcl_last_error() { return (int)cudaGetLastError(); }
