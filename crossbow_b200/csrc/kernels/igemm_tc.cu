// Implicit-GEMM convolution / inner product on the 5th-generation tensor cores (tcgen05), tf32 operands, fp32
// accumulation in tensor memory.
//
//   D[128 x BN] (TMEM)  +=  A[128 x 32] (smem, gathered im2col rows)  *  B[BN x 32]^T (smem, filter rows)
//
// One CTA (128 threads) owns a 128-row tile of output positions and up to 256 output channels.  Per 32-wide
// reduction slice every thread gathers ONE row of A (its output position: 8 x 16-byte loads with on-the-fly
// (r,s,c) bookkeeping, zero fill for padding) and a share of B straight into the canonical K-major, no-swizzle
// UMMA layout in shared memory ([16-byte k-chunk][row][16 B]; core matrix = 8 rows x 16 B, stride between 8-row
// groups 128 B, stride between k-chunks = rows*16 B).  One thread then issues four tcgen05.mma (M128, N=BN, K8,
// kind::tf32) and commits them to the stage's mbarrier; a 3-4 stage ring lets the gathers of the next slices run
// under the tensor-core work.  The epilogue reads the accumulator with tcgen05.ld (each warp its own 32 lanes),
// adds bias, applies ReLU, optionally accumulates onto the output and produces the per-channel sum / sum of
// squares that batch-norm needs, so a Conv -> BatchNorm pair reads the convolution output only once more.
//
// fprop and dgrad share the kernel (dgrad = transposed gather over dY with the (C,R,S,K) weight copy).  Replaces
// cudnnConvolutionForward / BackwardData and cublasSgemm of the reference (clib-multigpu/kernels/cudnnconv.cu:96-124,
// cudnnconvgradient.cu:156-169, innerproduct.cu:133-169, innerproductgradient.cu:152).
// Every mbarrier wait is bounded; on expiry the CTA records XB_TIMEOUT_MBAR, skips its stores, releases its tensor
// memory and exits.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int BM = 128;       // rows per CTA = UMMA M
constexpr int BKF = 32;       // floats per reduction slice (8 chunks of 16 bytes)
constexpr int NTHREADS = 128;

struct TcProblem {
  int M, OH, OW, IH, IW, CR, NG, R, S, sh, sw, ph, pw, transposed, KG;
};

using namespace tc;

constexpr int F_RELU = 1, F_ACCUM = 2, F_STATS = 4;

template <int BN, int STAGES>
__global__ void __launch_bounds__(NTHREADS) igemm_tc_kernel(const float* __restrict__ A, const float* __restrict__ Bw,
                                                            const float* __restrict__ bias, float* __restrict__ Out,
                                                            float* __restrict__ stats, TcProblem g, int flags, int* status) {
  constexpr uint32_t A_STAGE = BM * BKF * 4, B_STAGE = BN * BKF * 4;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;     // power of two >= 32 (BN is 16,32,64,128,256)
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sA = smem;
  unsigned char* sB = smem + STAGES * A_STAGE;
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ float s_red[2 * BN];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&bar_empty[s], 1);
    mbar_init(&bar_done, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // this thread's A row (output position)
  const int m = m0 + tid;
  const bool row_ok = m < g.M;
  int oy = 0, ox = 0;
  long long a_base = 0;
  if (row_ok) {
    ox = m % g.OW; int t = m / g.OW; oy = t % g.OH; int n = t / g.OH;
    a_base = (long long)n * g.IH * g.IW * g.CR;
  }
  // running (r, s, c) of the first chunk of the next slice to be fetched
  int kr = 0, ks = 0, kc = 0;

  // Asynchronous 16-byte copies global -> shared (zero fill when the source size is 0), STAGES-1 slices ahead.
  auto fetch = [&](int kt) {
    const int s = kt % STAGES;
    const uint32_t dA = smem_u32(sA + s * A_STAGE) + tid * 16;
    int r = kr, ss = ks, c = kc;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float* src = A;
      uint32_t bytes = 0;
      if (row_ok && r < g.R) {
        int iy, ix; bool ok;
        if (!g.transposed) {
          iy = oy * g.sh - g.ph + r; ix = ox * g.sw - g.pw + ss;
          ok = iy >= 0 && iy < g.IH && ix >= 0 && ix < g.IW;
        } else {
          int ty = oy + g.ph - r, tx = ox + g.pw - ss;
          ok = ty >= 0 && tx >= 0 && (ty % g.sh == 0) && (tx % g.sw == 0);
          iy = ty / g.sh; ix = tx / g.sw;
          ok = ok && iy < g.IH && ix < g.IW;
        }
        if (ok) { src = A + a_base + ((long long)iy * g.IW + ix) * g.CR + c; bytes = 16; }
      }
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dA + j * (BM * 16)), "l"(src), "r"(bytes) : "memory");
      c += 4;
      if (c >= g.CR) { c = 0; if (++ss >= g.S) { ss = 0; ++r; } }
    }
    kr = r; ks = ss; kc = c;
    const uint32_t dB = smem_u32(sB + s * B_STAGE);
    const int k0 = kt * BKF;
#pragma unroll
    for (int i = 0; i < (BN * 8 + NTHREADS - 1) / NTHREADS; ++i) {
      int idx = tid + i * NTHREADS;
      if (idx < BN * 8) {
        int row = idx % BN, chunk = idx / BN;
        int n = n0 + row, k = k0 + chunk * 4;
        const float* src = Bw;
        uint32_t bytes = 0;
        if (n < g.NG && k < g.KG) { src = Bw + (long long)n * g.KG + k; bytes = 16; }
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dB + (chunk * BN + row) * 16), "l"(src), "r"(bytes) : "memory");
      }
    }
  };

  const int ktiles = (g.KG + BKF - 1) / BKF;
  bool alive = true;
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    if (t < ktiles) fetch(t);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    const int s = kt % STAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");     // this thread's share of slice kt has landed
    fence_async_smem();
    __syncthreads();                                                         // ... and everybody else's
    // warp 0 re-converges (__syncwarp) before any of its lanes goes on to poll a barrier: a lane that is suspended in
    // mbarrier.try_wait must never share a warp with the lane that still has to issue the MMAs
    if (warp == 0) {
     if (lane == 0 && alive) {
      tc_fence_after();
      const uint32_t a0 = smem_u32(sA + s * A_STAGE), b0 = smem_u32(sB + s * B_STAGE);
#pragma unroll
      for (int k4 = 0; k4 < BKF / 8; ++k4) {
        uint64_t ad = make_desc(a0 + k4 * 2 * (BM * 16), BM * 16, 128);
        uint64_t bd = make_desc(b0 + k4 * 2 * (BN * 16), BN * 16, 128);
        umma_tf32(tmem, ad, bd, IDESC, (kt > 0 || k4 > 0) ? 1u : 0u);
      }
      umma_commit(&bar_empty[s]);
     }
     __syncwarp();
    }
    // refill the stage that slice kt-1 used (its MMAs were committed one iteration ago)
    const int nt = kt + STAGES - 1;
    if (nt < ktiles) {
      if (kt >= 1 && alive) {
        const int ps = (kt - 1) % STAGES;
        if (!mbar_wait(&bar_empty[ps], (uint32_t)(((kt - 1) / STAGES) & 1))) { alive = false; s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
      }
      fetch(nt);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (warp == 0) {
    if (lane == 0 && alive) umma_commit(&bar_done);
    __syncwarp();
  }
  if (alive && !mbar_wait(&bar_done, 0)) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
  tc_fence_after();
  __syncthreads();
  const bool abort_all = s_abort != 0;

  // ---- epilogue: warp w owns TMEM lanes 32w..32w+31 = rows m0+32w+lane ----
  if (flags & F_STATS) { for (int i = tid; i < 2 * BN; i += NTHREADS) s_red[i] = 0.f; }
  __syncthreads();
  if (!abort_all) {
    const int row = m0 + warp * 32 + lane;
    const bool ok = row < g.M;
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      float* orow = Out + (long long)row * g.NG + n0 + c0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n = n0 + c0 + j;
        float x = v[j];
        if (bias && n < g.NG) x += bias[n];
        if (flags & F_RELU) x = fmaxf(x, 0.f);
        if ((flags & F_ACCUM) && ok && n < g.NG) x += orow[j];
        v[j] = (ok && n < g.NG) ? x : 0.f;
      }
      if (ok) {
        if (n0 + c0 + 16 <= g.NG && ((g.NG & 3) == 0)) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(orow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (n0 + c0 + j < g.NG) orow[j] = v[j];
        }
      }
      if (flags & F_STATS) {
        float sq[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) sq[j] = v[j] * v[j];
        int col;
        float sx = warp_colsum16(v, lane, col), sqq = warp_colsum16(sq, lane, col);
        if (lane < 16) { atomicAdd(&s_red[c0 + col], sx); atomicAdd(&s_red[BN + c0 + col], sqq); }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if ((flags & F_STATS) && !abort_all) {
    for (int i = tid; i < BN; i += NTHREADS) {
      int n = n0 + i;
      if (n < g.NG) { atomicAdd(&stats[n], s_red[i]); atomicAdd(&stats[g.NG + n], s_red[BN + i]); }
    }
  }
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

template <int BN, int STAGES>
int launch_tc(const float* A, const float* Bw, const float* bias, float* Out, float* stats, const TcProblem& g, int flags, int* status,
              cudaStream_t st) {
  constexpr int smem = STAGES * (BM + BN) * BKF * 4;
  dim3 grid(xb_ceil_div(g.M, BM), xb_ceil_div(g.NG, BN));
  igemm_tc_kernel<BN, STAGES><<<grid, NTHREADS, smem, st>>>(A, Bw, bias, Out, stats, g, flags, status);
  return (int)cudaGetLastError();
}

int dispatch_tc(const float* A, const float* Bw, const float* bias, float* Out, float* stats, const TcProblem& g, int flags, int* status,
                cudaStream_t st) {
  if (g.NG <= 16) return launch_tc<16, 4>(A, Bw, bias, Out, stats, g, flags, status, st);
  if (g.NG <= 32) return launch_tc<32, 4>(A, Bw, bias, Out, stats, g, flags, status, st);
  if (g.NG <= 64) return launch_tc<64, 4>(A, Bw, bias, Out, stats, g, flags, status, st);
  if (g.NG <= 128) return launch_tc<128, 4>(A, Bw, bias, Out, stats, g, flags, status, st);
  return launch_tc<256, 3>(A, Bw, bias, Out, stats, g, flags, status, st);
}

template <int BN, int STAGES>
int configure_tc() {
  return (int)cudaFuncSetAttribute(igemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * (BM + BN) * BKF * 4);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

XB_API int xb_conv3x3_slab_supported(const XbConvGeom* g, int which);
XB_API int xb_conv3x3_slab_init();
XB_API int xb_conv3x3_slab(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which,
                           int flags, int* status, cudaStream_t st, const XbBnFuse* bnf);
XB_API int xb_conv3x3_wgrad_slab(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st);
static int g_use_slab = 3;
static int g_use_tma = 1;
XB_API int xb_gemm_tma_init();
XB_API int xb_conv_wgrad_simt(const float*, const float*, float*, const XbConvGeom*, cudaStream_t);
XB_API int xb_conv1x1_tma_supported(const XbConvGeom* g, int which);
XB_API int xb_conv1x1_tma(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which, int flags,
                          int* status, cudaStream_t st, const XbBnFuse* bnf);
XB_API int xb_conv1x1_wgrad_tma(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st);
// 1: 1x1 convolutions run on the TMA-fed GEMM kernel where it applies (else the gather kernel).  For A/B comparisons.
XB_API void xb_tc_set_tma(int on) { g_use_tma = on; }
XB_API int xb_conv_tma_supported(const XbConvGeom* g, int which);
XB_API int xb_conv_tma(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which, int flags,
                       int* status, cudaStream_t st, const XbBnFuse* bnf);
// R x S stride-1 convolutions with at least this many reduction channels run as a TMA implicit GEMM, narrower ones on the
// slab kernel (one staged copy of the input serves all taps, which wins while the filter bank is small).
static int g_tma_conv_min = 32;
XB_API void xb_tc_set_tma_conv_min(int c) { g_tma_conv_min = c; }
// bit 0: 3x3/stride-1 fprop + dgrad use the slab kernel (else the generic gather kernel); bit 1: the tensor-core weight
// gradient kernel is used where it applies (else CUDA cores).  For A/B comparisons.
XB_API void xb_tc_set_slab(int mask) { g_use_slab = mask; }

XB_API long long xb_conv_im2col_scratch(const XbConvGeom* g, int which);
// Bytes of scratch if the forward pass (which 0) or the weight gradient (which 2) of this layer should run as patch
// matrix + GEMM: that is, when no direct tensor-core kernel covers it.  0 otherwise.
XB_API long long xb_conv_im2col_wanted(const XbConvGeom* g, int which) {
  if (!g_use_tma) return 0;
  if (which == 0) {
    if ((g_use_slab & 1) && xb_conv3x3_slab_supported(g, 0)) return 0;
    if (xb_conv1x1_tma_supported(g, 0)) return 0;
    if ((g->R > 1 || g->S > 1) && g->C >= g_tma_conv_min && xb_conv_tma_supported(g, 0)) return 0;
  } else if (which == 2) {
    if (xb_conv1x1_tma_supported(g, 2)) return 0;
    if ((g_use_slab & 2) && xb_conv3x3_slab_supported(g, 2)) return 0;
  } else {
    return 0;
  }
  if (g->P == 1 && g->Q == 1 && g->H == 1 && g->W == 1) return 0;   // inner products keep to the GEMM-shaped kernels
  const long long b = xb_conv_im2col_scratch(g, which);
  return b <= (1ll << 30) ? b : 0;
}

// Opt in to the large dynamic shared-memory carve-outs once per process, outside any stream capture.
XB_API int xb_tc_init() {
  int e;
  if ((e = xb_conv3x3_slab_init())) return e;
  if ((e = xb_gemm_tma_init())) return e;
  if ((e = configure_tc<16, 4>())) return e;
  if ((e = configure_tc<32, 4>())) return e;
  if ((e = configure_tc<64, 4>())) return e;
  if ((e = configure_tc<128, 4>())) return e;
  if ((e = configure_tc<256, 3>())) return e;
  return 0;
}

// which: 0 fprop, 1 dgrad, 2 wgrad.  The tensor-core path needs a reduction-channel count that is a multiple of 4
// (16-byte gathers); everything else runs on the CUDA-core kernels.
XB_API int xb_tc_supported(const XbConvGeom* g, int which) {
  if (which == 0) return (g->C % 4 == 0) ? 1 : 0;
  if (which == 1) return (g->K % 4 == 0) ? 1 : 0;
  if (g_use_tma && xb_conv1x1_tma_supported(g, 2)) return 1;
  return (g_use_slab & 2) && xb_conv3x3_slab_supported(g, 2) ? 1 : 0;
}

XB_API int xb_conv_fprop_tc(const float* X, const float* W, const float* bias, float* Y, float* stats, const XbConvGeom* cg, int flags,
                            int* status, cudaStream_t st) {
  if (!aligned16(X) || !aligned16(W) || !aligned16(Y) || cg->C % 4) return -XB_BAD_ARG;
  if (g_use_tma && (cg->R > 1 || cg->S > 1) && cg->C >= g_tma_conv_min && xb_conv_tma_supported(cg, 0)) {
    const int r = xb_conv_tma(X, W, bias, Y, stats, cg, 0, flags, status, st, nullptr);
    if (r != -XB_BAD_ARG) return r;
  }
  if ((g_use_slab & 1) && xb_conv3x3_slab_supported(cg, 0)) return xb_conv3x3_slab(X, W, bias, Y, stats, cg, 0, flags, status, st, nullptr);
  if (g_use_tma && xb_conv1x1_tma_supported(cg, 0)) {
    const int r = xb_conv1x1_tma(X, W, bias, Y, stats, cg, 0, flags, status, st, nullptr);
    if (r != -XB_BAD_ARG) return r;                      // (tensor map refused: fall back to the gather kernel)
  }
  TcProblem g;
  g.M = cg->N * cg->P * cg->Q; g.OH = cg->P; g.OW = cg->Q; g.IH = cg->H; g.IW = cg->W; g.CR = cg->C; g.NG = cg->K;
  g.R = cg->R; g.S = cg->S; g.sh = cg->sh; g.sw = cg->sw; g.ph = cg->ph; g.pw = cg->pw; g.transposed = 0; g.KG = cg->R * cg->S * cg->C;
  return dispatch_tc(X, W, bias, Y, stats, g, flags, status, st);
}
// 1 if the kernel that xb_conv_dgrad_tc picks for this layer can also produce the batch-norm backward sums of the layer
// that owns dX (XbBnFuse).  It must visit every element of dX, which rules out the strided 1x1 form.
XB_API int xb_conv_dgrad_fuses_bn(const XbConvGeom* cg) {
  if (cg->K % 4 || cg->C % 4) return 0;
  if (g_use_tma && (cg->R > 1 || cg->S > 1) && cg->K >= g_tma_conv_min && xb_conv_tma_supported(cg, 1)) return 1;
  if ((g_use_slab & 1) && xb_conv3x3_slab_supported(cg, 1)) return 1;
  if (g_use_tma && cg->sh == 1 && xb_conv1x1_tma_supported(cg, 1)) return 1;
  return 0;
}
XB_API int xb_conv_dgrad_tc(const float* dY, const float* Wt, float* dX, const XbConvGeom* cg, int accumulate, int* status, cudaStream_t st,
                            const XbBnFuse* bnf) {
  if (bnf && bnf->sums && !xb_conv_dgrad_fuses_bn(cg)) return -XB_BAD_ARG;
  if (!aligned16(dY) || !aligned16(Wt) || !aligned16(dX) || cg->K % 4) return -XB_BAD_ARG;
  if (g_use_tma && (cg->R > 1 || cg->S > 1) && cg->K >= g_tma_conv_min && xb_conv_tma_supported(cg, 1)) {
    const int r = xb_conv_tma(dY, Wt, nullptr, dX, nullptr, cg, 1, accumulate ? F_ACCUM : 0, status, st, bnf);
    if (r != -XB_BAD_ARG) return r;
  }
  if ((g_use_slab & 1) && xb_conv3x3_slab_supported(cg, 1)) return xb_conv3x3_slab(dY, Wt, nullptr, dX, nullptr, cg, 1, accumulate ? F_ACCUM : 0, status, st, bnf);
  if (g_use_tma && xb_conv1x1_tma_supported(cg, 1)) {
    const int r = xb_conv1x1_tma(dY, Wt, nullptr, dX, nullptr, cg, 1, accumulate ? F_ACCUM : 0, status, st, bnf);
    if (r != -XB_BAD_ARG) return r;
  }
  TcProblem g;
  g.M = cg->N * cg->H * cg->W; g.OH = cg->H; g.OW = cg->W; g.IH = cg->P; g.IW = cg->Q; g.CR = cg->K; g.NG = cg->C;
  g.R = cg->R; g.S = cg->S; g.sh = cg->sh; g.sw = cg->sw; g.ph = cg->ph; g.pw = cg->pw; g.transposed = 1; g.KG = cg->R * cg->S * cg->K;
  return dispatch_tc(dY, Wt, nullptr, dX, nullptr, g, accumulate ? F_ACCUM : 0, status, st);
}
XB_API int xb_conv_wgrad_tc(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st) {
  if (!aligned16(dY) || !aligned16(X)) return -XB_BAD_ARG;
  if (g_use_tma && xb_conv1x1_tma_supported(cg, 2)) {
    const int r = xb_conv1x1_wgrad_tma(dY, X, dW, cg, status, st);
    return r != -XB_BAD_ARG ? r : xb_conv_wgrad_simt(dY, X, dW, cg, st);
  }
  if (!xb_conv3x3_slab_supported(cg, 2)) return -XB_BAD_ARG;
  return xb_conv3x3_wgrad_slab(dY, X, dW, cg, status, st);
}
