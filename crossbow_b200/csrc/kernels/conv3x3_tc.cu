// 3x3 / stride 1 / pad 1 convolution (forward and data gradient) on tcgen05 without any im2col traffic.
//
// Idea: walk the output in a "padded position space" in which every image has one zero row on top (shared with the
// image above: H+1 rows) and one zero column on each side (W+2 columns).  In that space the nine taps of a 3x3 filter
// are nine CONSTANT shifts of one linear index: source = position + (r-1)*(W+2) + (s-1).  A CTA therefore stages one
// contiguous slab of 128 + 2*(W+2) + 2 positions x C channels in shared memory ONCE, laid out as
// [16-byte channel chunk][position][16 B], which is exactly the canonical K-major no-swizzle UMMA operand layout
// (core matrix = 8 positions x 16 B).  The A operand of tap (r,s) is then the same slab with its descriptor start
// address advanced by (r*(W+2)+s)*16 bytes: nine descriptors, one copy of the data, zero redundant global reads
// (the gather formulation re-reads every input element nine times and spends ~700 instructions per thread per
// reduction slice on address arithmetic).  The filter bank is staged once as [chunk][output channel][16 B].
// One elected thread issues 9*C/8 tcgen05.mma (M128 x N x K8, tf32) into a TMEM accumulator and commits; the epilogue
// drops the rows that fall on padding positions, adds bias / ReLU / accumulation, and produces the batch-norm sums.
//
// dgrad of such a convolution is the same computation over dY with the taps mirrored and the (C,R,S,K) weight copy.
#include "common.cuh"
#include "tc_ptx.cuh"

using namespace tc;

namespace {

constexpr int BM = 128, NTHREADS = 128;
constexpr int F_RELU = 1, F_ACCUM = 2, F_STATS = 4;

struct SlabProblem {
  int N, H, W, C, K;      // C = reduction channels, K = output channels (already swapped for dgrad)
  int mirrored;           // 1: dgrad (tap (r,s) uses the weights of tap (2-r,2-s))
  long long positions;    // N*(H+1)*(W+2)
};

template <int BN>
__global__ void __launch_bounds__(NTHREADS) conv3x3_slab_kernel(const float* __restrict__ X, const float* __restrict__ Wb,
                                                                const float* __restrict__ bias, float* __restrict__ Out,
                                                                float* __restrict__ stats, SlabProblem g, int flags, int* status) {
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ float s_red[2 * BN];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int PW = g.W + 2, PR = g.H + 1;
  const int S = BM + 2 * PW + 2;                      // slab length in positions
  const int CQ = g.C >> 2;                            // 16-byte chunks per position
  const uint32_t plane = (uint32_t)S * 16u;           // bytes per chunk plane of the slab
  unsigned char* sSlab = smem;
  unsigned char* sB = smem + (size_t)CQ * plane;      // [9*CQ chunks][BN rows][16 B]
  const long long q0 = (long long)blockIdx.x * BM;
  const long long qs = q0 - PW - 1;
  const int n0 = blockIdx.y * BN;

  if (tid == 0) {
    mbar_init(&bar_done, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);

  // ---- stage the slab: one (position, chunk) = 16 bytes per copy, zero fill for padding positions ----
  const uint32_t slab_u32 = smem_u32(sSlab);
  for (int j = tid; j < S; j += NTHREADS) {
    const long long p = qs + j;
    const float* src = X;
    uint32_t bytes = 0;
    if (p >= 0 && p < g.positions) {
      int xx = (int)(p % PW); long long t = p / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
      if (yy >= 1 && xx >= 1 && xx <= g.W) { src = X + (((long long)n * g.H + (yy - 1)) * g.W + (xx - 1)) * g.C; bytes = 16; }
    }
    for (int c = 0; c < CQ; ++c)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(slab_u32 + c * plane + j * 16), "l"(src + (bytes ? c * 4 : 0)), "r"(bytes) : "memory");
  }
  // ---- stage the filter bank: chunk index = tap*CQ + c ; row = output channel ----
  const uint32_t b_u32 = smem_u32(sB);
  const int KG = 9 * g.C;
  for (int idx = tid; idx < 9 * CQ * BN; idx += NTHREADS) {
    int row = idx % BN, chunk = idx / BN;
    int tap = chunk / CQ, c = chunk - tap * CQ;
    int wtap = g.mirrored ? (8 - tap) : tap;
    int n = n0 + row;
    const float* src = Wb;
    uint32_t bytes = 0;
    if (n < g.K) { src = Wb + (long long)n * KG + wtap * g.C + c * 4; bytes = 16; }
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(b_u32 + (chunk * BN + row) * 16), "l"(src), "r"(bytes) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // The whole of warp 0 takes this branch and re-converges at the __syncwarp below BEFORE any of its lanes starts to
  // poll the completion barrier: lanes that spin in mbarrier.try_wait (which may suspend them) while a sibling lane of
  // the same warp still has instructions to issue would starve that lane.
  if (warp == 0) {
   if (lane == 0) {
    const int k8s = g.C >> 3;
    uint32_t acc = 0;
    for (int tap = 0; tap < 9; ++tap) {
      const int r = tap / 3, s = tap - 3 * r;
      const uint32_t a_tap = slab_u32 + (uint32_t)(r * PW + s) * 16u;
      for (int k8 = 0; k8 < k8s; ++k8) {
        uint64_t ad = make_desc(a_tap + (uint32_t)(2 * k8) * plane, plane, 128);
        uint64_t bd = make_desc(b_u32 + (uint32_t)((tap * CQ + 2 * k8) * BN) * 16u, BN * 16, 128);
        umma_tf32(tmem, ad, bd, IDESC, acc);
        acc = 1;
      }
    }
    umma_commit(&bar_done);
   }
   __syncwarp();
  }
  if (!mbar_wait(&bar_done, 0)) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
  tc_fence_after();
  if (flags & F_STATS) { for (int i = tid; i < 2 * BN; i += NTHREADS) s_red[i] = 0.f; }
  __syncthreads();
  const bool abort_all = s_abort != 0;

  if (!abort_all) {
    const long long q = q0 + warp * 32 + lane;
    bool ok = false;
    long long opix = 0;
    if (q < g.positions) {
      int xx = (int)(q % PW); long long t = q / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
      ok = yy >= 1 && xx >= 1 && xx <= g.W;
      opix = ((long long)n * g.H + (yy - 1)) * g.W + (xx - 1);
    }
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      float* orow = Out + opix * g.K + n0 + c0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n = n0 + c0 + j;
        float x = v[j];
        if (bias && n < g.K) x += bias[n];
        if (flags & F_RELU) x = fmaxf(x, 0.f);
        if ((flags & F_ACCUM) && ok && n < g.K) x += orow[j];
        v[j] = (ok && n < g.K) ? x : 0.f;
      }
      if (ok) {
        if (n0 + c0 + 16 <= g.K && ((g.K & 3) == 0)) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(orow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (n0 + c0 + j < g.K) orow[j] = v[j];
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
      if (n < g.K) { atomicAdd(&stats[n], s_red[i]); atomicAdd(&stats[g.K + n], s_red[BN + i]); }
    }
  }
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}


// ---- weight gradient of a 3x3 / stride 1 / pad 1 convolution -------------------------------------------------------------
// dW[k][tap][c] = sum over positions of dY[pos][k] * X[pos + shift(tap)][c].  The reduction runs over POSITIONS, and in the
// slab layout [16-byte channel chunk][position][16 B] a group of 8 consecutive positions x 4 channels is one contiguous
// 128-byte core matrix - exactly the canonical MN-major no-swizzle operand (MN = channel, K = position; stride between
// channel chunks = SBO, between groups of 8 positions = LBO = 128 B).  So the SAME two slabs serve as operands again:
//   A = dY tile   (M = output channels, padded to 128 by zero planes)      B = X slab shifted by the tap (N = input channels)
// A persistent CTA walks position tiles, accumulating nine [128 x BN] products (one per tap) in 9*BN TMEM columns, and
// adds its partial dW to global memory once at the end.
template <int BN>
__global__ void __launch_bounds__(NTHREADS) conv3x3_wgrad_slab_kernel(const float* __restrict__ dY, const float* __restrict__ X,
                                                                      float* __restrict__ dW, SlabProblem g, int ntiles, int* status) {
  constexpr uint32_t TMEM_COLS = 9 * BN <= 256 ? 256 : 512;
  // M = 128, N = BN, both operands MN-major (bits 15 and 16)
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int PW = g.W + 2, PR = g.H + 1;
  const int S = BM + 2 * PW + 2;
  const int KQ = g.K >> 2;                             // real 16-byte chunks of dY (output channels / 4)
  const int c0 = blockIdx.y * BN;                      // first input channel of this CTA's N tile
  constexpr uint32_t planeA = BM * 16u;                // dY tile: 32 planes x 128 positions x 16 B
  const uint32_t planeB = (uint32_t)S * 16u;
  unsigned char* sA = smem;
  unsigned char* sB = smem + 32 * planeA;              // [BN/4 planes][S positions][16 B]
  const uint32_t a_u32 = smem_u32(sA), b_u32 = smem_u32(sB);

  if (tid == 0) { mbar_init(&bar_done, 1); s_abort = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);
  // planes of A beyond the real output channels stay zero for the whole kernel
  for (int i = tid; i < (32 - KQ) * BM; i += NTHREADS) reinterpret_cast<float4*>(sA + (size_t)KQ * planeA)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  uint32_t phase = 0;
  bool first = true, alive = true;
  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long q0 = (long long)tile * BM, qs = q0 - PW - 1;
    if (!first) {                                       // the previous tile's MMAs must have consumed shared memory
      if (alive && !mbar_wait(&bar_done, phase)) { alive = false; s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
      phase ^= 1;
      __syncthreads();
    }
    // dY tile: position m = tid, zero for padding positions
    {
      const long long p = q0 + tid;
      const float* src = dY; uint32_t bytes = 0;
      if (p < g.positions) {
        int xx = (int)(p % PW); long long t = p / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
        if (yy >= 1 && xx >= 1 && xx <= g.W) { src = dY + (((long long)n * g.H + (yy - 1)) * g.W + (xx - 1)) * g.K; bytes = 16; }
      }
      for (int c = 0; c < KQ; ++c)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_u32 + c * planeA + tid * 16), "l"(src + (bytes ? c * 4 : 0)), "r"(bytes) : "memory");
    }
    // X slab (with halo), only this CTA's BN input channels
    for (int j = tid; j < S; j += NTHREADS) {
      const long long p = qs + j;
      const float* src = X; uint32_t bytes = 0;
      if (p >= 0 && p < g.positions) {
        int xx = (int)(p % PW); long long t = p / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
        if (yy >= 1 && xx >= 1 && xx <= g.W) { src = X + (((long long)n * g.H + (yy - 1)) * g.W + (xx - 1)) * g.C + c0; bytes = 16; }
      }
      for (int c = 0; c < BN / 4; ++c) {
        uint32_t b = (bytes && c0 + c * 4 < g.C) ? 16u : 0u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(b_u32 + c * planeB + j * 16), "l"(src + (b ? c * 4 : 0)), "r"(b) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
      if (lane == 0 && alive) {
        tc_fence_after();
        for (int tap = 0; tap < 9; ++tap) {
          const int r = tap / 3, s = tap - 3 * r;
          const uint32_t shift = (uint32_t)(r * PW + s) * 16u;
#pragma unroll 4
          for (int j = 0; j < BM / 8; ++j) {             // 8 positions per MMA
            uint64_t ad = make_desc(a_u32 + j * 128, 128, planeA);
            uint64_t bd = make_desc(b_u32 + shift + j * 128, 128, planeB);
            umma_tf32(tmem + tap * BN, ad, bd, IDESC, (first && j == 0) ? 0u : 1u);
          }
        }
        umma_commit(&bar_done);
      }
      __syncwarp();
    }
    first = false;
  }
  if (!first && alive && !mbar_wait(&bar_done, phase)) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
  tc_fence_after();
  __syncthreads();
  if (!s_abort && !first) {
    const int k = warp * 32 + lane;                      // output channel = TMEM lane
    const bool warp_has_rows = warp * 32 < g.K;          // whole-warp condition: tcgen05.ld is warp-collective
    if (warp_has_rows) {
      for (int tap = 0; tap < 9; ++tap)
#pragma unroll
        for (int cc = 0; cc < BN; cc += 16) {
          float v[16];
          tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(tap * BN + cc), v);
          if (k < g.K) {
            float* o = dW + ((long long)k * 9 + tap) * g.C + c0 + cc;
#pragma unroll
            for (int j = 0; j < 16; ++j) if (c0 + cc + j < g.C) atomicAdd(o + j, v[j]);
          }
        }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

inline size_t wgrad_smem_bytes(int W, int BN) { return (size_t)32 * BM * 16 + (size_t)(BN / 4) * (BM + 2 * (W + 2) + 2) * 16; }

inline size_t slab_smem_bytes(int W, int C, int BN) {
  size_t S = BM + 2 * (W + 2) + 2;
  return (size_t)(C / 4) * S * 16 + (size_t)9 * (C / 4) * BN * 16;
}
constexpr size_t kSmemLimit = 200 * 1024;


// ---- the same convolution for wide layers: the reduction channels are walked in chunks of CC through a two-stage ring ---
// Per stage: CC/4 planes of the slab + the matching slice of all nine filter taps.  While the tensor core consumes
// chunk i from one stage, cp.async fills the other with chunk i+1; an mbarrier per stage (tcgen05.commit) tells when
// the stage may be overwritten.  Everything else (padded position space, shifted descriptors, epilogue) is as above.
template <int BN, int CC>
__global__ void __launch_bounds__(NTHREADS) conv3x3_slab_pipe_kernel(const float* __restrict__ X, const float* __restrict__ Wb,
                                                                     const float* __restrict__ bias, float* __restrict__ Out,
                                                                     float* __restrict__ stats, SlabProblem g, int flags, int* status) {
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr int CQ = CC / 4;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ float s_red[2 * BN];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int PW = g.W + 2, PR = g.H + 1;
  const int S = BM + 2 * PW + 2;
  const uint32_t plane = (uint32_t)S * 16u;
  const uint32_t slab_bytes = (uint32_t)CQ * plane, b_bytes = 9u * CQ * BN * 16u;
  const uint32_t stage_bytes = (slab_bytes + b_bytes + 127u) & ~127u;
  const long long q0 = (long long)blockIdx.x * BM;
  const long long qs = q0 - PW - 1;
  const int n0 = blockIdx.y * BN;
  const int nchunks = g.C / CC;
  const int KG = 9 * g.C;
  const uint32_t smem_base = smem_u32(smem);

  if (tid == 0) {
    mbar_init(&bar_empty[0], 1); mbar_init(&bar_empty[1], 1); mbar_init(&bar_done, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);

  // per-thread slab positions are the same for every chunk: decode them once (at most 3 positions per thread)
  const float* pos_src[3]; int pos_j[3]; int npos = 0;
  for (int j = tid; j < S && npos < 3; j += NTHREADS) {
    const long long p = qs + j;
    const float* src = nullptr;
    if (p >= 0 && p < g.positions) {
      int xx = (int)(p % PW); long long t = p / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
      if (yy >= 1 && xx >= 1 && xx <= g.W) src = X + (((long long)n * g.H + (yy - 1)) * g.W + (xx - 1)) * g.C;
    }
    pos_src[npos] = src; pos_j[npos] = j; ++npos;
  }
  auto fetch = [&](int ch) {
    const uint32_t st = smem_base + (uint32_t)(ch & 1) * stage_bytes;
    const int cbase = ch * CC;
    for (int i = 0; i < npos; ++i) {
      const float* src = pos_src[i];
#pragma unroll
      for (int c = 0; c < CQ; ++c)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(st + c * plane + pos_j[i] * 16), "l"(src ? src + cbase + c * 4 : X), "r"(src ? 16u : 0u) : "memory");
    }
    const uint32_t sb = st + slab_bytes;
    for (int idx = tid; idx < 9 * CQ * BN; idx += NTHREADS) {
      int row = idx % BN, chunk = idx / BN;
      int tap = chunk / CQ, c = chunk - tap * CQ;
      int wtap = g.mirrored ? (8 - tap) : tap;
      int n = n0 + row;
      const bool ok = n < g.K;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(sb + (chunk * BN + row) * 16),
                   "l"(ok ? Wb + (long long)n * KG + wtap * g.C + cbase + c * 4 : Wb), "r"(ok ? 16u : 0u) : "memory");
    }
  };
  fetch(0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  if (nchunks > 1) fetch(1);
  asm volatile("cp.async.commit_group;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  bool alive = true;
  for (int ch = 0; ch < nchunks; ++ch) {
    const int s = ch & 1;
    asm volatile("cp.async.wait_group 1;" ::: "memory");        // everything but the most recent group has landed
    fence_async_smem();
    __syncthreads();
    if (warp == 0) {
      if (lane == 0 && alive) {
        tc_fence_after();
        const uint32_t st = smem_base + (uint32_t)s * stage_bytes, sb = st + slab_bytes;
        for (int tap = 0; tap < 9; ++tap) {
          const int r = tap / 3, sx = tap - 3 * r;
          const uint32_t a_tap = st + (uint32_t)(r * PW + sx) * 16u;
#pragma unroll
          for (int k8 = 0; k8 < CC / 8; ++k8) {
            uint64_t ad = make_desc(a_tap + (uint32_t)(2 * k8) * plane, plane, 128);
            uint64_t bd = make_desc(sb + (uint32_t)((tap * CQ + 2 * k8) * BN) * 16u, BN * 16, 128);
            umma_tf32(tmem, ad, bd, IDESC, (ch > 0 || tap > 0 || k8 > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bar_empty[s]);
      }
      __syncwarp();
    }
    if (ch + 2 < nchunks) {
      if (alive && !mbar_wait(&bar_empty[s], (uint32_t)((ch >> 1) & 1))) { alive = false; s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
      fetch(ch + 2);
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
  if (flags & F_STATS) { for (int i = tid; i < 2 * BN; i += NTHREADS) s_red[i] = 0.f; }
  __syncthreads();
  const bool abort_all = s_abort != 0;

  if (!abort_all) {
    const long long q = q0 + warp * 32 + lane;
    bool ok = false;
    long long opix = 0;
    if (q < g.positions) {
      int xx = (int)(q % PW); long long t = q / PW; int yy = (int)(t % PR); int n = (int)(t / PR);
      ok = yy >= 1 && xx >= 1 && xx <= g.W;
      opix = ((long long)n * g.H + (yy - 1)) * g.W + (xx - 1);
    }
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      float* orow = Out + opix * g.K + n0 + c0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        int n = n0 + c0 + j;
        float x = v[j];
        if (bias && n < g.K) x += bias[n];
        if (flags & F_RELU) x = fmaxf(x, 0.f);
        if ((flags & F_ACCUM) && ok && n < g.K) x += orow[j];
        v[j] = (ok && n < g.K) ? x : 0.f;
      }
      if (ok) {
        if (n0 + c0 + 16 <= g.K && ((g.K & 3) == 0)) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(orow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (n0 + c0 + j < g.K) orow[j] = v[j];
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
      if (n < g.K) { atomicAdd(&stats[n], s_red[i]); atomicAdd(&stats[g.K + n], s_red[BN + i]); }
    }
  }
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

inline size_t pipe_smem_bytes(int W, int CC, int BN) {
  size_t S = BM + 2 * (W + 2) + 2;
  size_t stage = ((size_t)(CC / 4) * S * 16 + (size_t)9 * (CC / 4) * BN * 16 + 127) & ~(size_t)127;
  return 2 * stage;
}

template <int BN>
int launch_slab(const float* X, const float* Wb, const float* bias, float* Out, float* stats, const SlabProblem& g, int flags, int* status,
                cudaStream_t st) {
  size_t smem = slab_smem_bytes(g.W, g.C, BN);
  dim3 grid((unsigned)((g.positions + BM - 1) / BM), (unsigned)((g.K + BN - 1) / BN));
  conv3x3_slab_kernel<BN><<<grid, NTHREADS, smem, st>>>(X, Wb, bias, Out, stats, g, flags, status);
  return (int)cudaGetLastError();
}
inline int pick_bn(int K) { return K <= 16 ? 16 : K <= 32 ? 32 : K <= 64 ? 64 : K <= 128 ? 128 : 256; }
// Output-channel tile: as wide as the layer allows, but narrower when the grid would leave SMs idle (small feature maps:
// every CTA then stages fewer filters and the per-CTA latency chain gets shorter) or when shared memory would overflow.
inline int choose_bn(long long positions, int W, int Cred, int Kout) {
  int bn = pick_bn(Kout);
  const long long tiles_m = (positions + BM - 1) / BM;
  while (bn > 16 && tiles_m * ((Kout + bn - 1) / bn) < 2 * 148) bn >>= 1;
  while (bn > 16 && slab_smem_bytes(W, Cred, bn) > kSmemLimit) bn >>= 1;
  return bn;
}

}  // namespace

template <int BN>
int launch_pipe(const float* X, const float* Wb, const float* bias, float* Out, float* stats, const SlabProblem& g, int flags, int* status,
                cudaStream_t st) {
  size_t smem = pipe_smem_bytes(g.W, 16, BN);
  dim3 grid((unsigned)((g.positions + BM - 1) / BM), (unsigned)((g.K + BN - 1) / BN));
  conv3x3_slab_pipe_kernel<BN, 16><<<grid, NTHREADS, smem, st>>>(X, Wb, bias, Out, stats, g, flags, status);
  return (int)cudaGetLastError();
}
inline int choose_pipe_bn(long long positions, int W, int Kout) {
  int bn = Kout <= 16 ? 16 : Kout <= 32 ? 32 : Kout <= 64 ? 64 : 128;
  const long long tiles_m = (positions + BM - 1) / BM;
  while (bn > 16 && tiles_m * ((Kout + bn - 1) / bn) < 148) bn >>= 1;
  while (bn > 16 && pipe_smem_bytes(W, 16, bn) > kSmemLimit) bn >>= 1;
  return bn;
}

// 1 if the slab kernel covers this geometry in direction `which` (0 fprop, 1 dgrad)
XB_API int xb_conv3x3_slab_supported(const XbConvGeom* g, int which) {
  if (g->R != 3 || g->S != 3 || g->sh != 1 || g->sw != 1 || g->ph != 1 || g->pw != 1) return 0;
  if (which == 2) return (g->C % 16 == 0 && g->K % 4 == 0 && g->K <= 128 && wgrad_smem_bytes(g->W, 32) <= kSmemLimit) ? 1 : 0;
  int Cred = which == 0 ? g->C : g->K, Kout = which == 0 ? g->K : g->C;
  if (Cred % 8 || Kout % 4) return 0;
  const long long positions = (long long)g->N * (g->H + 1) * (g->W + 2);
  if (slab_smem_bytes(g->W, Cred, choose_bn(positions, g->W, Cred, Kout)) <= kSmemLimit) return 1;
  // (the pipelined kernel keeps at most three slab positions per thread in registers: S = 130 + 2*(W+2) <= 384)
  return (Cred % 16 == 0 && g->W <= 120 && pipe_smem_bytes(g->W, 16, choose_pipe_bn(positions, g->W, Kout)) <= kSmemLimit) ? 1 : 0;
}
XB_API int xb_conv3x3_slab_init() {
  int e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_pipe_kernel<16, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_pipe_kernel<32, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_pipe_kernel<64, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_slab_pipe_kernel<128, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_slab_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_slab_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  return 0;
}
// dW (K,3,3,C) must hold the value to accumulate onto (normally zero).
XB_API int xb_conv3x3_wgrad_slab(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st) {
  SlabProblem g;
  g.N = cg->N; g.H = cg->H; g.W = cg->W; g.C = cg->C; g.K = cg->K; g.mirrored = 0;
  g.positions = (long long)cg->N * (cg->H + 1) * (cg->W + 2);
  const int ntiles = (int)((g.positions + BM - 1) / BM);
  const int BN = cg->C <= 16 ? 16 : 32;
  dim3 grid((unsigned)(ntiles < 148 ? ntiles : 148), (unsigned)((cg->C + BN - 1) / BN));
  if (grid.y > 1 && grid.x * grid.y > 296) grid.x = 296 / grid.y;
  if (BN == 16) conv3x3_wgrad_slab_kernel<16><<<grid, NTHREADS, wgrad_smem_bytes(g.W, 16), st>>>(dY, X, dW, g, ntiles, status);
  else          conv3x3_wgrad_slab_kernel<32><<<grid, NTHREADS, wgrad_smem_bytes(g.W, 32), st>>>(dY, X, dW, g, ntiles, status);
  return (int)cudaGetLastError();
}

// which: 0 fprop (In = X, Wb = weights (K,3,3,C)), 1 dgrad (In = dY, Wb = transposed copy (C,3,3,K), output dX)
XB_API int xb_conv3x3_slab(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which,
                           int flags, int* status, cudaStream_t st) {
  SlabProblem g;
  g.N = cg->N; g.H = cg->H; g.W = cg->W;
  g.C = which == 0 ? cg->C : cg->K; g.K = which == 0 ? cg->K : cg->C;
  g.mirrored = which;
  g.positions = (long long)cg->N * (cg->H + 1) * (cg->W + 2);
  if (slab_smem_bytes(g.W, g.C, choose_bn(g.positions, g.W, g.C, g.K)) > kSmemLimit) {
    switch (choose_pipe_bn(g.positions, g.W, g.K)) {
      case 16: return launch_pipe<16>(In, Wb, bias, Out, stats, g, flags, status, st);
      case 32: return launch_pipe<32>(In, Wb, bias, Out, stats, g, flags, status, st);
      case 64: return launch_pipe<64>(In, Wb, bias, Out, stats, g, flags, status, st);
      default: return launch_pipe<128>(In, Wb, bias, Out, stats, g, flags, status, st);
    }
  }
  switch (choose_bn(g.positions, g.W, g.C, g.K)) {
    case 16: return launch_slab<16>(In, Wb, bias, Out, stats, g, flags, status, st);
    case 32: return launch_slab<32>(In, Wb, bias, Out, stats, g, flags, status, st);
    case 64: return launch_slab<64>(In, Wb, bias, Out, stats, g, flags, status, st);
    case 128: return launch_slab<128>(In, Wb, bias, Out, stats, g, flags, status, st);
    default: return launch_slab<256>(In, Wb, bias, Out, stats, g, flags, status, st);
  }
}
