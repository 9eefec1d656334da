// Symmetric heap plumbing: device allocations that every rank of the box can
// address.  Each rank allocates the same number of bytes with cudaMalloc,
// exports a CUDA IPC handle, and opens the handles of its peers; kernels then
// receive a device array of `world` base pointers and issue loads, stores and
// reductions to peers over NVLink.  (The reference's equivalent plumbing is the
// ZeroMQ socket set of include/client.hpp:38-42 plus the server table of
// include/kv_def.hpp:23-24.)
#include "common.cuh"
#include <string.h>

PCL_API int pcl_symm_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 256);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes ? bytes : 256);
  if (e != cudaSuccess) return (int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return (int)e; }
  static_assert(sizeof(h) == 64, "ipc handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}

PCL_API int pcl_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

PCL_API int pcl_symm_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

PCL_API int pcl_symm_free(void* ptr) { return (int)cudaFree(ptr); }

PCL_API int pcl_device_sync() { return (int)cudaDeviceSynchronize(); }

PCL_API const char* pcl_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }
