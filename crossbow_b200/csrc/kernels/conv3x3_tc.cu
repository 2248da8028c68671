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
constexpr int F_RELU = 1, F_ACCUM = 2, F_STATS = 4, F_BNBWD = 8;   // F_BNBWD: `stats` receives batch-norm backward sums (XbBnFuse)

struct SlabProblem {
  int N, H, W, C, K;      // C = reduction channels, K = output channels (already swapped for dgrad)
  int mirrored;           // 1: dgrad (tap (r,s) uses the weights of tap (2-r,2-s))
  long long positions;    // N*(H+1)*(W+2)
};

template <int BN>
__global__ void __launch_bounds__(NTHREADS) conv3x3_slab_kernel(const float* __restrict__ X, const float* __restrict__ Wb,
                                                                const float* __restrict__ bias, float* __restrict__ Out,
                                                                float* __restrict__ stats, SlabProblem g, int flags, int* status, XbBnFuse bn) {
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
  xb_pdl_wait();                                       // nothing above reads or writes global memory
  xb_pdl_launch();
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
  if (flags & (F_STATS | F_BNBWD)) { for (int i = tid; i < 2 * BN; i += NTHREADS) s_red[i] = 0.f; }
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
      if (flags & (F_STATS | F_BNBWD)) {
        float sq[16];
        if (flags & F_BNBWD) {                             // v = final dy of a normalisation layer: its backward sums
          const long long off = opix * g.K + n0 + c0;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = n0 + c0 + j;
            float dz = 0.f, t = 0.f;
            if (ok && n < g.K) {
              dz = (bn.relu && !(bn.y[off + j] > 0.f)) ? 0.f : v[j];
              t = dz * (bn.x[off + j] - bn.mean[n]) * bn.istd[n];
            }
            v[j] = dz; sq[j] = t;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) sq[j] = v[j] * v[j];
        }
        int col;
        float sx = warp_colsum16(v, lane, col), sqq = warp_colsum16(sq, lane, col);
        if (lane < 16) { atomicAdd(&s_red[c0 + col], sx); atomicAdd(&s_red[BN + c0 + col], sqq); }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if ((flags & (F_STATS | F_BNBWD)) && !abort_all) {
    for (int i = tid; i < BN; i += NTHREADS) {
      int n = n0 + i;
      if (n < g.K) { atomicAdd(&stats[n], s_red[i]); atomicAdd(&stats[g.K + n], s_red[BN + i]); }
    }
  }
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}


// ---- weight gradient of a 3x3 / stride 1 / pad 1 convolution -------------------------------------------------------------
// dW[k][r][s][c] = sum over positions p of dY[p][k] * X[p + r*(W+2) + s][c]  (padded position space, slab index).
// The reduction runs over POSITIONS while both tensors are stored position-major with the channels contiguous, i.e. both
// operands are "MN-major".  For 32-bit operands tcgen05 accepts exactly one MN-major shared-memory layout: 128-byte rows
// (32 channels of one position), four rows per 512-byte atom, the 32-byte chunks of a row XOR-ed with bits 7..8 of the
// absolute address (layout type 1, "128-byte swizzle with 32-byte base"); SBO is the stride between groups of four rows,
// LBO the stride between groups of 32 MN elements.  The swizzle works on absolute address bits, so a descriptor whose
// start is advanced by whole rows still reads a consistently swizzled slab: measured on B200, and the basis of this
// kernel.  Operands:
//   A = the X slab.  M = 128 = 4 groups x 32 channels with LBO = ONE ROW (128 B): group g re-reads the slab one
//       position further on, so the four groups are the taps s = 0, 1, 2 (and one unused) of filter row r.
//   B = the dY tile, N = output channels, 32 per plane (LBO = plane stride).
// One M128 x N x K8 MMA per filter row and 8 positions therefore covers three taps; 48 MMAs per 128-position tile.
// The three accumulators (one per filter row) live in 3*N TMEM columns across all tiles a persistent CTA walks; a two-stage
// cp.async ring overlaps the loads of tile i+1 with the MMAs of tile i.  At the end TMEM lane (s, c) adds its 3*N values to
// dW - 32 consecutive lanes hit 32 consecutive floats.
constexpr int WG_THREADS = 512;                        // many warps: the cp.async loads are latency-bound per warp
template <int NK>
__global__ void __launch_bounds__(WG_THREADS) conv3x3_wgrad_mn_kernel(const float* __restrict__ dY, const float* __restrict__ X,
                                                                    float* __restrict__ dW, SlabProblem g, int ntiles, int* status) {
  constexpr int NP = (NK + 31) / 32;                   // 32-channel planes of the dY tile
  constexpr int YQ = NK / 4;                           // 16-byte chunks per dY position
  constexpr uint32_t TMEM_COLS = 3 * NK <= 64 ? 64 : 3 * NK <= 128 ? 128 : 3 * NK <= 256 ? 256 : 512;
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(NK >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint64_t LAYOUT = 1ull << 61;
  constexpr uint32_t yplane = BM * 128u;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_free[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int PW = g.W + 2, PR = g.H + 1;
  const int S = (BM + 2 * PW + 4 + 3) & ~3;            // slab rows: the tile, two filter rows of halo, the group shift
  const int c0 = blockIdx.y * 32, k0 = blockIdx.z * NK;
  const int xq = (g.C - c0 >= 32 ? 32 : g.C - c0) >> 2;  // valid 16-byte chunks per slab row
  const uint32_t xbytes = (uint32_t)S * 128u, stage_bytes = xbytes + NP * yplane;
  const uint32_t base_u32 = smem_u32(smem);
  if (tid == 0) { mbar_init(&bar_free[0], 3); mbar_init(&bar_free[1], 3); s_abort = 0; asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  xb_pdl_wait();                                       // nothing above reads or writes global memory
  xb_pdl_launch();
  if (warp == 0) tmem_alloc(&s_tmem, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // Pixel index (n*H + y)*W + x of every slab row of a tile, -1 for padding: computed once per tile with 32-bit
  // arithmetic so that the copy loops below carry no divisions.  Two tables, alternating with the stages.
  int* s_pix = reinterpret_cast<int*>(smem + 2 * stage_bytes);
  const int npos = (int)g.positions;
  auto load_tile = [&](int tile, int stage) {
    const uint32_t sbase = base_u32 + (uint32_t)stage * stage_bytes;
    int* pix = s_pix + stage * S;
    const int q0 = tile * BM, qs = q0 - PW - 1;
    for (int j = tid; j < S; j += WG_THREADS) {
      const int p = qs + j;
      int v = -1;
      if (p >= 0 && p < npos) {
        const int t = p / PW, xx = p - t * PW, n = t / PR, yy = t - n * PR;
        if (yy >= 1 && xx >= 1 && xx <= g.W) v = (n * g.H + (yy - 1)) * g.W + (xx - 1);
      }
      pix[j] = v;
    }
    __syncthreads();
    {                                                    // X slab: eight threads per row, one 16-byte chunk each
      const uint32_t q = (uint32_t)tid & 7u;
      if ((int)q < xq) {
        const float* xsrc = X + c0 + q * 4;
        for (int j = tid >> 3; j < S; j += WG_THREADS / 8) {
          const int v = pix[j];
          const float* src = v >= 0 ? xsrc + (long long)v * g.C : X;
          const uint32_t dst = sbase + (uint32_t)j * 128u + (((q >> 1) ^ ((uint32_t)j & 3u)) << 5) + (q & 1u) * 16u;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(v >= 0 ? 16u : 0u) : "memory");
        }
      }
    }
    {                                                    // dY tile: YQ threads per row
      const uint32_t q = (uint32_t)tid % YQ, qq = q & 7u;
      const bool kin = k0 + (int)q * 4 < g.K;
      const float* ysrc = dY + k0 + q * 4;
      const uint32_t ybase = sbase + xbytes + (q >> 3) * yplane;
      for (int t = tid / YQ; t < BM; t += WG_THREADS / YQ) {
        const int v = kin ? pix[t + PW + 1] : -1;
        const float* src = v >= 0 ? ysrc + (long long)v * g.K : dY;
        const uint32_t dst = ybase + (uint32_t)t * 128u + (((qq >> 1) ^ ((uint32_t)t & 3u)) << 5) + (qq & 1u) * 16u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(v >= 0 ? 16u : 0u) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // Called by all threads after the loads of iteration `it` have landed (and a __syncthreads): one lane issues the MMAs.
  auto issue_tile = [&](int it, bool alive) {
    // The three filter rows accumulate into three independent TMEM regions, and THREE threads (lane 0 of warps 0..2) issue
    // them: one thread sustains only about one tcgen05.mma per 70 cycles, far below what the tensor pipe needs for these
    // small-N products, and issue streams of different threads overlap.  Each thread commits its own MMAs; the stage
    // barrier counts three arrivals.
    if (warp < 3) {
      if (lane == 0 && alive) {
        tc_fence_after();
        const uint32_t sbase = base_u32 + (uint32_t)(it & 1) * stage_bytes;
        const int r = warp;
#pragma unroll 4
        for (int j = 0; j < BM / 8; ++j) {
          const uint64_t bd = make_desc(sbase + xbytes + (uint32_t)j * 1024u, yplane, 512) | LAYOUT;
          const uint64_t ad = make_desc(sbase + (uint32_t)(r * PW) * 128u + (uint32_t)j * 1024u, 128, 512) | LAYOUT;
          umma_tf32(tmem + (uint32_t)(r * NK), ad, bd, IDESC, (it == 0 && j == 0) ? 0u : 1u);
        }
        umma_commit(&bar_free[it & 1]);
      }
      __syncwarp();
    }
  };

  const int my_tiles = blockIdx.x < ntiles ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  bool alive = true;
  for (int it = 0; it < my_tiles; ++it) {
    if (it >= 2) {                                       // the MMAs of tile it-2 must have consumed this stage
      if (alive && !mbar_wait(&bar_free[it & 1], (uint32_t)(((it >> 1) - 1) & 1))) { alive = false; s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
    }
    load_tile((int)blockIdx.x + it * (int)gridDim.x, it & 1);
    if (it >= 1) {
      asm volatile("cp.async.wait_group 1;" ::: "memory");
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      issue_tile(it - 1, alive);
    }
  }
  if (my_tiles > 0) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    issue_tile(my_tiles - 1, alive);
    const int last = my_tiles - 1;
    if (alive && !mbar_wait(&bar_free[last & 1], (uint32_t)((last >> 1) & 1))) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
  }
  tc_fence_after();
  __syncthreads();
  if (!s_abort && my_tiles > 0 && (warp & 3) < 3) {      // TMEM lane quadrant (warp & 3) = filter column s, lane = input channel
    const int sx = warp & 3, c = c0 + lane;
    for (int ch = warp >> 2; ch < 3 * NK / 16; ch += WG_THREADS / 128) {   // 16-column chunks, dealt to the warps of a quadrant
      const int r = (ch * 16) / NK, n0 = (ch * 16) % NK;
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(sx * 32) << 16) + (uint32_t)(ch * 16), v);
      if (c < g.C) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int kk = k0 + n0 + j;
          if (kk < g.K) atomicAdd(dW + ((long long)kk * 9 + r * 3 + sx) * g.C + c, v[j]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

inline size_t wgrad_smem_bytes(int W, int NK) {
  size_t S = (BM + 2 * (W + 2) + 4 + 3) & ~3;
  return 2 * (S * 128 + (size_t)((NK + 31) / 32) * BM * 128) + 2 * S * sizeof(int);
}

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
                                                                     float* __restrict__ stats, SlabProblem g, int flags, int* status, XbBnFuse bn) {
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
  xb_pdl_wait();                                       // nothing above reads or writes global memory
  xb_pdl_launch();
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
  if (flags & (F_STATS | F_BNBWD)) { for (int i = tid; i < 2 * BN; i += NTHREADS) s_red[i] = 0.f; }
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
      if (flags & (F_STATS | F_BNBWD)) {
        float sq[16];
        if (flags & F_BNBWD) {                             // v = final dy of a normalisation layer: its backward sums
          const long long off = opix * g.K + n0 + c0;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = n0 + c0 + j;
            float dz = 0.f, t = 0.f;
            if (ok && n < g.K) {
              dz = (bn.relu && !(bn.y[off + j] > 0.f)) ? 0.f : v[j];
              t = dz * (bn.x[off + j] - bn.mean[n]) * bn.istd[n];
            }
            v[j] = dz; sq[j] = t;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) sq[j] = v[j] * v[j];
        }
        int col;
        float sx = warp_colsum16(v, lane, col), sqq = warp_colsum16(sq, lane, col);
        if (lane < 16) { atomicAdd(&s_red[c0 + col], sx); atomicAdd(&s_red[BN + c0 + col], sqq); }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if ((flags & (F_STATS | F_BNBWD)) && !abort_all) {
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
                cudaStream_t st, const XbBnFuse& bn) {
  size_t smem = slab_smem_bytes(g.W, g.C, BN);
  dim3 grid((unsigned)((g.positions + BM - 1) / BM), (unsigned)((g.K + BN - 1) / BN));
  xb_launch(conv3x3_slab_kernel<BN>, grid, dim3(NTHREADS), smem, st, X, Wb, bias, Out, stats, g, flags, status, bn);
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

// Output channels per CTA of the weight-gradient kernel: as many as fit in two shared-memory stages.
inline int choose_wgrad_nk(int W, int K) {
  int nk = K <= 16 ? 16 : K <= 32 ? 32 : K <= 64 ? 64 : 128;
  while (nk > 16 && wgrad_smem_bytes(W, nk) > kSmemLimit) nk >>= 1;
  return nk;
}

}  // namespace

template <int BN>
int launch_pipe(const float* X, const float* Wb, const float* bias, float* Out, float* stats, const SlabProblem& g, int flags, int* status,
                cudaStream_t st, const XbBnFuse& bn) {
  size_t smem = pipe_smem_bytes(g.W, 16, BN);
  dim3 grid((unsigned)((g.positions + BM - 1) / BM), (unsigned)((g.K + BN - 1) / BN));
  xb_launch(conv3x3_slab_pipe_kernel<BN, 16>, grid, dim3(NTHREADS), smem, st, X, Wb, bias, Out, stats, g, flags, status, bn);
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
  if (which == 2) return (g->C % 4 == 0 && g->K % 4 == 0 && (long long)g->N * (g->H + 1) * (g->W + 2) < (1ll << 30) && wgrad_smem_bytes(g->W, choose_wgrad_nk(g->W, g->K)) <= kSmemLimit) ? 1 : 0;
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
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_mn_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_mn_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_mn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if ((e = (int)cudaFuncSetAttribute(conv3x3_wgrad_mn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  return 0;
}
// Upper bound on the CTAs of one weight-gradient launch (each adds a full partial dW to global memory at its end).
static int g_wgrad_ctas = 148;
XB_API void xb_conv3x3_wgrad_set_ctas(int n) { g_wgrad_ctas = n > 0 ? n : 148; }
// dW (K,3,3,C) must hold the value to accumulate onto (normally zero).
XB_API int xb_conv3x3_wgrad_slab(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st) {
  SlabProblem g;
  g.N = cg->N; g.H = cg->H; g.W = cg->W; g.C = cg->C; g.K = cg->K; g.mirrored = 0;
  g.positions = (long long)cg->N * (cg->H + 1) * (cg->W + 2);
  const int ntiles = (int)((g.positions + BM - 1) / BM);
  const int NK = choose_wgrad_nk(g.W, g.K);
  const unsigned gy = (unsigned)((g.C + 31) / 32), gz = (unsigned)((g.K + NK - 1) / NK);
  // Few, long-lived CTAs: each one ends with 9*C*K atomic adds and holds tensor memory and ~85 KB of shared memory while it
  // runs.  Measured end to end: 74 CTAs are best for the small layers (ResNet-32: +6 % images/s over 296), 111-148 for the
  // large ones (ResNet-50).
  const int cap = ((long long)ntiles * gy * gz < 700) ? g_wgrad_ctas / 2 : g_wgrad_ctas;
  int gx = cap / (int)(gy * gz);
  if (gx < 1) gx = 1;
  if (gx > ntiles) gx = ntiles;
  dim3 grid((unsigned)gx, gy, gz);
  const size_t smem = wgrad_smem_bytes(g.W, NK);
  switch (NK) {
    case 16: xb_launch(conv3x3_wgrad_mn_kernel<16>, grid, dim3(WG_THREADS), smem, st, dY, X, dW, g, ntiles, status); break;
    case 32: xb_launch(conv3x3_wgrad_mn_kernel<32>, grid, dim3(WG_THREADS), smem, st, dY, X, dW, g, ntiles, status); break;
    case 64: xb_launch(conv3x3_wgrad_mn_kernel<64>, grid, dim3(WG_THREADS), smem, st, dY, X, dW, g, ntiles, status); break;
    default: xb_launch(conv3x3_wgrad_mn_kernel<128>, grid, dim3(WG_THREADS), smem, st, dY, X, dW, g, ntiles, status); break;
  }
  return (int)cudaGetLastError();
}

// which: 0 fprop (In = X, Wb = weights (K,3,3,C)), 1 dgrad (In = dY, Wb = transposed copy (C,3,3,K), output dX)
XB_API int xb_conv3x3_slab(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which,
                           int flags, int* status, cudaStream_t st, const XbBnFuse* bnf) {
  XbBnFuse bn{};
  if (bnf && bnf->sums) { bn = *bnf; stats = bnf->sums; flags = (flags & ~F_STATS) | F_BNBWD; }
  SlabProblem g;
  g.N = cg->N; g.H = cg->H; g.W = cg->W;
  g.C = which == 0 ? cg->C : cg->K; g.K = which == 0 ? cg->K : cg->C;
  g.mirrored = which;
  g.positions = (long long)cg->N * (cg->H + 1) * (cg->W + 2);
  if (slab_smem_bytes(g.W, g.C, choose_bn(g.positions, g.W, g.C, g.K)) > kSmemLimit) {
    switch (choose_pipe_bn(g.positions, g.W, g.K)) {
      case 16: return launch_pipe<16>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
      case 32: return launch_pipe<32>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
      case 64: return launch_pipe<64>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
      default: return launch_pipe<128>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
    }
  }
  switch (choose_bn(g.positions, g.W, g.C, g.K)) {
    case 16: return launch_slab<16>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
    case 32: return launch_slab<32>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
    case 64: return launch_slab<64>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
    case 128: return launch_slab<128>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
    default: return launch_slab<256>(In, Wb, bias, Out, stats, g, flags, status, st, bn);
  }
}

// ---- data gradient of a 3x3 / stride 2 / pad 1 convolution ---------------------------------------------------------------
// dX[h] = sum_r dY_up[h + 1 - r] w[r] with dY_up[2p] = dY[p] and zeros in between: exactly the stride-1 data gradient over the
// zero-inserted output gradient.  A small kernel writes dY_up (input resolution, K channels) into caller-provided scratch and
// the slab kernel above does the rest on the tensor core.
namespace {
__global__ void upsample2_zero_kernel(const float* __restrict__ dY, float* __restrict__ up, int N, int P, int Q, int H, int W, int K4) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)N * H * W * K4;
  if (idx >= total) return;
  const int k4 = (int)(idx % K4); long long t = idx / K4;
  const int w = (int)(t % W); t /= W;
  const int h = (int)(t % H); const int n = (int)(t / H);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!(h & 1) && !(w & 1) && (h >> 1) < P && (w >> 1) < Q)
    v = reinterpret_cast<const float4*>(dY)[(((long long)n * P + (h >> 1)) * Q + (w >> 1)) * K4 + k4];
  reinterpret_cast<float4*>(up)[idx] = v;
}
inline XbConvGeom stride1_of(const XbConvGeom* g) {
  XbConvGeom s = *g;
  s.sh = 1; s.sw = 1; s.P = g->H; s.Q = g->W;
  return s;
}
}  // namespace

// bytes of scratch if this layer's data gradient can run this way, else 0
XB_API long long xb_conv3x3_s2_dgrad_scratch(const XbConvGeom* g) {
  if (g->R != 3 || g->S != 3 || g->sh != 2 || g->sw != 2 || g->ph != 1 || g->pw != 1) return 0;
  if ((g->H & 1) || (g->W & 1) || g->P != g->H / 2 || g->Q != g->W / 2 || (g->K & 3)) return 0;
  XbConvGeom s = stride1_of(g);
  if (!xb_conv3x3_slab_supported(&s, 1)) return 0;
  return (long long)g->N * g->H * g->W * g->K * 4;
}
XB_API int xb_conv3x3_s2_dgrad(const float* dY, const float* Wt, float* dX, const XbConvGeom* cg, int accumulate, float* scratch, int* status,
                               cudaStream_t st, const XbBnFuse* bnf) {
  if (!scratch || !xb_conv3x3_s2_dgrad_scratch(cg)) return -XB_BAD_ARG;
  const long long total = (long long)cg->N * cg->H * cg->W * (cg->K / 4);
  upsample2_zero_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(dY, scratch, cg->N, cg->P, cg->Q, cg->H, cg->W, cg->K / 4);
  int e = (int)cudaGetLastError();
  if (e) return e;
  XbConvGeom s = stride1_of(cg);
  return xb_conv3x3_slab(scratch, Wt, nullptr, dX, nullptr, &s, 1, accumulate ? F_ACCUM : 0, status, st, bnf);
}
