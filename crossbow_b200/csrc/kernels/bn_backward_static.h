// Batch-norm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which always goes through cuDNN and its own buffer pools).
// It exists for hosts that drive the library from a context where cudaMalloc is off limits: code running inside
// another framework's memory pool, inside a CUDA-graph-capturing region of the caller, in a real-time loop that must not
// take the allocator lock, or in a process whose device memory is fully pre-partitioned.  The regular entry point
// (xb_bn_backward) needs a caller-provided, zeroed scratch vector of 2*C floats for the per-channel sums of the
// gradient; here that scratch lives in a fixed array inside the library instead.
//
//   * The array holds XB_BN_STATIC_MAX_CHANNELS channels (2 * 4096 floats = 32 KB).  Every GPU on which the library is
//     loaded carries it until the process exits.  A call with more channels is refused with XB_BN_STATIC_TOO_MANY_CHANNELS
//     (and one line on stderr); nothing is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device current.
//     Make that first call outside any stream capture.  Host threads may make their first calls concurrently (the looked-up
//     address is kept in an atomic).  Later calls only enqueue work on `stream`: one memset of the
//     part of the array that is used (the sums must start from zero) and the two backward kernels.
//   * All calls share the one array, which keeps the previous call's sums.  Two calls that overlap on the GPU (different
//     streams, or different host threads without ordering) race on it; serialise them.
//   * Arguments and results are those of xb_bn_backward minus the scratch pointer: dgamma / dbeta are accumulated (+=).
//   * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define XB_BN_STATIC_MAX_CHANNELS 4096
#define XB_BN_STATIC_TOO_MANY_CHANNELS (-1001)
#define XB_BN_STATIC_BAD_ARGUMENT (-1002)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, one of the codes above, or a positive cudaError_t.
int xb_bn_backward_static(const float* dy, const float* x, const float* y, const float* save_mean, const float* save_invstd,
                          const float* gamma, float* dx, float* dres, float* dgamma, float* dbeta, int M, int C, int relu,
                          int accum_dx, int accum_dres, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
