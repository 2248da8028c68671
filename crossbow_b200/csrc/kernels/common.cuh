// Shared definitions for the sm_100a kernels: geometry structs, per-task parameter block, status word.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define XB_API extern "C" __attribute__((visibility("default")))

// Convolution / inner-product geometry.  Activations are channels-last (N,H,W,C); weights are (K,R,S,C).
// An inner product is the R=S=H=W=1 case.
struct XbConvGeom {
  int N, H, W, C;      // input
  int K, R, S;         // filters
  int P, Q;            // output spatial extent
  int sh, sw, ph, pw;  // stride / padding
};

// Batch-norm backward sums produced by the epilogue of the kernel that writes the gradient dy of a normalisation layer
// (the data gradient of the next convolution): sums[c] += dz, sums[C + c] += dz * (x - mean[c]) * istd[c] with
// dz = dy masked by the layer's fused ReLU (y > 0).  x = the layer's input, y = its output; all of dy's shape.
struct XbBnFuse {
  const float* x; const float* y; const float* mean; const float* istd;
  float* sums;
  int relu;
};

// Values that change from task to task.  They live in device memory (one block per learner) and are refreshed
// by a host-to-device copy in front of the task's kernels, so a captured CUDA graph never bakes them in.
struct XbTaskParams {
  float lr;          // learning rate of this task (positive)
  float momentum;
  float weight_decay;
  float bn_factor;   // running-statistics blend factor: 1-fraction, or 1/(1+updates) for CMA
  float clip;        // gradient-norm threshold, <0 = off
  float alpha;       // averaging constant
  unsigned int task_id;
  unsigned int seed_lo, seed_hi;
  int training;
  int l1;            // 1 = L1 regularisation
  int nesterov;
};

// Error/status codes written by kernels that can give up (bounded waits) or detect bad arguments.
enum XbStatus : int { XB_OK = 0, XB_TIMEOUT_FLAG = 1, XB_TIMEOUT_MBAR = 2, XB_BAD_ARG = 3 };

#define XB_CUDA_CHECK(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return (int)_e;                    \
  } while (0)

// ---- programmatic dependent launch -------------------------------------------------------------------------------------
// A task is a chain of ~150 kernels of 5-15 us each, every one of which needs the results of the one before.  With a plain
// launch the next kernel's blocks are only scheduled once the previous grid has drained and its memory has been flushed;
// launched with the programmatic-serialisation attribute (an edge of that kind in a captured graph) they are scheduled
// while the previous grid's last blocks still run, set up what does not depend on it (shared-memory copies of their
// arguments, barriers, descriptor prefetch) and then sit in xb_pdl_wait() until the previous grid has completed and its
// writes are visible.  Rules for a kernel launched through xb_launch:
//   * no access to global memory that another kernel of the stream produces, or consumes and this one overwrites, before
//     xb_pdl_wait();
//   * xb_pdl_wait() is executed by every thread that touches such memory afterwards (put it on a block-uniform path);
//   * xb_pdl_launch() AFTER the wait: the kernel after this one may then be scheduled as soon as all blocks of this one
//     have started, never more than one kernel ahead.
// Both instructions do nothing in a kernel that was launched the plain way.
__device__ __forceinline__ void xb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void xb_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_xb_pdl;                                     // defined in train_ops.cu; xb_set_pdl()

template <class... KArgs, class... Args>
static inline cudaError_t xb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = g_xb_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int xb_ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---- Philox4x32-10 (bit-identical to crossbow_b200/utils/philox.py) ----
__device__ __forceinline__ uint4 xb_philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}
__device__ __forceinline__ float xb_u24(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }
