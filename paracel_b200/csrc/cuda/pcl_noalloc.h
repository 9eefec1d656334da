// Entry point for callers that are not allowed to allocate device memory.
//
// This has no counterpart in the reference (douban/paracel has no GPU code and
// no notion of device allocation); it exists for embedders of this library.
//
// Who needs it: a process that gave all of its device memory to one arena
// when it started (an inference or feature server, a database engine), code
// that runs as a plug-in inside another framework's memory pool, and tight
// control loops that cannot afford the device-wide synchronisation cudaMalloc
// and cudaFree imply.  Such callers still own the inputs and outputs; what they
// cannot provide is the kernel's scratch space, so this variant keeps it in a
// fixed array that is part of the loaded library image.
//
//   pcl_lr_dense_grad_noalloc computes exactly what pcl_lr_dense_grad computes
//   (g[d] = sum over rows of (y - h(theta.x)) * x and the summed loss, h =
//   sigmoid when `logistic` is non-zero, identity otherwise) but takes no
//   scratch and no counter argument.
//
// Limits and rules:
//   * blocks * d + 2 * blocks + 4 must not exceed PCL_NOALLOC_MAX_FLOATS
//     (1 Mi floats = 4 MiB; with the default 296 blocks that is d <= 3540);
//     larger requests are refused with cudaErrorInvalidValue and a message that
//     pcl_lr_dense_grad_noalloc_error() returns.
//   * Every GPU that loads the library holds those 4 MiB until the process ends.
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current).  Make that first call
//     outside of any stream capture.
//   * All calls on a device share the array and it keeps what the last call
//     left there.  The call clears the one word that has to start at zero
//     itself.  Two calls whose kernels can overlap on the GPU (different
//     streams without an ordering between them) race on the array: order them.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.
//     The 4 MiB themselves are taken by the CUDA runtime when it loads this
//     library's device code on a GPU; with lazy module loading that can be as
//     late as the first call on that GPU (or any earlier kernel of this
//     library there).  An embedder that hands the rest of the memory to an
//     arena should make that first call before it sizes the arena.
//   * Host threads: calls from several host threads are serialised by a lock
//     inside the function (set-up and launch), so threads that drive different
//     devices may call at the same time; pcl_lr_dense_grad_noalloc_error()
//     returns the message of the calling thread's own last call.  Every
//     non-zero return code leaves a message.  The rule on overlapping kernels
//     of one device above still holds between threads.
#pragma once
#include <cuda_runtime.h>

#define PCL_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int pcl_lr_dense_grad_noalloc(const float* X, const float* y, const float* theta, long long n,
                              int d, int logistic, float* g, double* loss, int blocks,
                              cudaStream_t stream);

const char* pcl_lr_dense_grad_noalloc_error(void);

#ifdef __cplusplus
}
#endif
