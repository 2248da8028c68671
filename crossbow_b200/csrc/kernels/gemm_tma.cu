// 1x1 convolutions (and any plain GEMM over position-major tensors) on TMA + tcgen05.
//
// A 1x1 convolution over NHWC data is a GEMM whose operands already sit in memory in the shape the tensor core wants, so
// nothing is gathered: TMA (cp.async.bulk.tensor) drops swizzled operand tiles into shared memory, one elected thread
// issues tcgen05.mma into a TMEM accumulator, and eight epilogue warps drain it.  Warp roles in a 320-thread CTA:
//   warp 0      producer: waits for a free stage, arms its mbarrier with the byte count, issues the TMA loads
//   warp 1      tensor core: waits for a full stage, issues 4 x (M128 x BN x K8, tf32), tcgen05.commit frees the stage
//   warps 2..9  epilogue: wait for the accumulator, tcgen05.ld, bias / ReLU / accumulate / batch-norm sums, store; the two
//               warps of a TMEM lane quadrant take alternate 32-column blocks
// Two operand forms:
//   NT  D[m][n] = sum_k A[m][k] B[n][k]        (fprop: A = X, B = W (K,C);  dgrad: A = dY, B = W^T (C,K))
//       both operands K-major, 128-byte swizzle, 32 floats of K per stage.  A is described by a 3-D tensor map
//       (channel, column, row) so that a stride-2 convolution is the same kernel with doubled global strides.
//   CONV the NT form as an implicit GEMM for R x S / stride 1 / "same" convolutions: the reduction index is (tap, channel
//       block); the A tile of a tap is ONE 4-D TMA box (channel, column, row, image) whose start coordinate is shifted by
//       the tap - rows and columns outside the image arrive as zeros from the TMA unit, so padding costs nothing and no
//       index arithmetic runs on the SM.  The data gradient is the same kernel over dY with the taps mirrored.
//   TN  D[m][n] += sum_p A[p][m] B[p][n]       (wgrad: A = dY, B = X, reduction over positions)
//       both operands MN-major in the "128-byte swizzle, 32-byte atom" layout - the one layout tcgen05 reads 32-bit
//       MN-major data from - written by TMA with the matching swizzle mode; 32 positions per stage; the position range is
//       split over gridDim.z and every CTA adds its partial product to D with vector reductions.
// A pipeline stage holds KC (1, 2 or 4) consecutive 32-float reduction blocks: the issuing thread pays a fixed ~500 cycles per
// stage for the barrier round trip (wait full, commit empty) whatever the tile, so narrow tiles want many MMAs per stage.
// Every wait is bounded; on expiry the CTA records XB_TIMEOUT_MBAR in *status, drains and exits.
#include <cuda.h>
#include "common.cuh"
#include "tc_ptx.cuh"

using namespace tc;

namespace {

constexpr int GT = 320;                                 // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two per TMEM lane quadrant)
// 32-column tiles have one 32-column epilogue block per TMEM lane quadrant: four epilogue warps, not eight
// (the weight-gradient form deals 16-column blocks to the two warps of a quadrant and always needs both)
__host__ __device__ constexpr int gemm_threads(int BN, int MODE) { return (BN <= 32 && MODE != 1) ? 192 : GT; }
constexpr int EPI_BYTES = 8 * 32 * 33 * 4;              // one 32 x 32 transpose block per epilogue warp
constexpr int MAX_STAGES = 8;
constexpr int G_RELU = 1, G_ACCUM = 2, G_STATS = 4, G_BNBWD = 8;   // G_BNBWD: `stats` receives batch-norm backward sums (XbBnFuse)
constexpr int G_SPLITK = 16;                            // NT: the reduction is split over gridDim.z; every CTA adds its partial tile to D
constexpr uint32_t A_BYTES = 128 * 128;                 // 128 rows (or 4 planes x 32 positions) x 128 B

struct GemmArgs {
  int M, N;            // NT: real output rows / columns.  TN: output rows (filters) / columns (input channels)
  int kblocks;         // NT: ceil(K / 32).  TN: ceil(positions / 32)
  int mvalid;          // NT: rows of one tile that exist (box columns x box rows <= 128)
  int c1_step, c2_step;  // NT: A coordinates of tile t are {k, t * c1_step, t * c2_step}
  int a_bytes;         // NT: bytes one A box delivers
  int ldd;             // floats between rows of D
  int stages;
  int kb_per_split;    // TN: position blocks per gridDim.z slice.  NT: reduction blocks per slice, 0 = no split (G_SPLITK)
  int planes2d;        // TN: the operands are rank-2 maps (channel, position) and every 32-channel plane is a load of its own
  // CONV: the A box is {32 channels, bw columns, bh rows, bn images}; tiles are numbered (image group, row group, column group)
  int c32, R, S, ph, pw, H, W, NI, bw, bh, bn, tiles_w, tiles_h, mirrored, krow;
  // NT with a strided output (data gradient of a stride-2 1x1 convolution): row m = (n, p, q) of the GEMM is written to
  // pixel (n, 2p, 2q) of an (oH, oW) image.  0 = rows are written where they are.
  int oP, oQ, oH, oW;
  // TN over a sub-sampled B (weight gradient of a stride-2 1x1 convolution): one reduction block = rpb output rows of Q
  // positions (ppb = rpb * Q <= 32); rows ppb..31 of every stage stay zero.  0 = 32 consecutive positions per block.
  int rpb, ppb;
  int kc;              // NT / CONV: 32-float reduction blocks per pipeline stage (1, 2 or 4); kblocks counts stages' worth
};

template <int BN, int MODE, int KC>
__global__ void __launch_bounds__(gemm_threads(BN, MODE)) gemm_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                      float* __restrict__ D, const float* __restrict__ bias, float* __restrict__ stats,
                                                      GemmArgs g, int flags, int* status, XbBnFuse bn) {
  constexpr int NTH = gemm_threads(BN, MODE);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t B_BYTES = BN * 128, STAGE = KC * (A_BYTES + B_BYTES);   // stage = [A sub-blocks][B sub-blocks]
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (MODE == 1 ? (3u << 15) : 0u) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], accum_bar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ float s_red[2 * BN];
  __shared__ long long s_rowoff[4][32];                  // float offset of every tile row in D, -1 for rows that do not exist

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, n0 = blockIdx.y * BN;
  const int stages = g.stages;
  const uint32_t base = smem_u32(smem);
  int kb0 = 0, kb1 = g.kblocks;
  if (MODE == 1 || (MODE == 0 && g.kb_per_split)) { kb0 = blockIdx.z * g.kb_per_split; kb1 = kb0 + g.kb_per_split < g.kblocks ? kb0 + g.kb_per_split : g.kblocks; }
  const int nkb = kb1 - kb0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  xb_pdl_wait();                                       // nothing above reads or writes global memory (the maps are arguments)
  xb_pdl_launch();
  if (warp == 1) tmem_alloc(&s_tmem, TMEM_COLS);
  for (int i = tid; i < 2 * BN; i += NTH) s_red[i] = 0.f;
  if (MODE == 1 && g.rpb) {                              // rows the boxes never write must read as zero
    const int words = stages * (int)(STAGE / 16);
    for (int i = tid; i < words; i += NTH) reinterpret_cast<float4*>(smem)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  if (nkb > 0) {
    if (warp == 0) {
      if (lane == 0) {
        // CONV: position of the tile and a running (filter row, filter column, channel block) counter - no divisions in the loop
        int wt = 0, ht = 0, nt = 0, cr = 0, cs = 0, ccb = 0;
        if (MODE == 2) { wt = tile % g.tiles_w; const int t2 = tile / g.tiles_w; ht = t2 % g.tiles_h; nt = t2 / g.tiles_h; }
        for (int i = 0; i < nkb; ++i) {
          const int s = i % stages, kb = kb0 + i;
          if (i >= stages && !mbar_wait(&empty_bar[s], (uint32_t)((i / stages) - 1) & 1u)) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); break; }
          const uint32_t sa = base + (uint32_t)s * STAGE, sb = sa + KC * A_BYTES;
          if (MODE == 0) {
            mbar_expect_tx(&full_bar[s], KC * ((uint32_t)g.a_bytes + B_BYTES));
#pragma unroll
            for (int u = 0; u < KC; ++u) {
              tma_load_3d(sa + u * A_BYTES, &tmA, (kb * KC + u) * 32, tile * g.c1_step, tile * g.c2_step, &full_bar[s]);
              tma_load_2d(sb + u * B_BYTES, &tmB, (kb * KC + u) * 32, n0, &full_bar[s]);
            }
          } else if (MODE == 2) {
            // step kb covers KC consecutive (tap, channel block) pairs of the reduction, in tap-major order
            mbar_expect_tx(&full_bar[s], KC * ((uint32_t)g.a_bytes + B_BYTES));
#pragma unroll
            for (int u = 0; u < KC; ++u) {
              const int tap = cr * g.S + cs, btap = g.mirrored ? g.R * g.S - 1 - tap : tap;
              tma_load_4d(sa + u * A_BYTES, &tmA, ccb * 32, wt * g.bw + cs - g.pw, ht * g.bh + cr - g.ph, nt * g.bn, &full_bar[s]);
              tma_load_2d(sb + u * B_BYTES, &tmB, btap * g.krow + ccb * 32, n0, &full_bar[s]);
              if (++ccb == g.c32) { ccb = 0; if (++cs == g.S) { cs = 0; ++cr; } }
            }
          } else if (g.rpb == 0 && !g.planes2d) {
            mbar_expect_tx(&full_bar[s], STAGE);
            tma_load_3d(sa, &tmA, 0, kb * 32, tile * 4, &full_bar[s]);
            tma_load_3d(sb, &tmB, 0, kb * 32, n0 >> 5, &full_bar[s]);
          } else if (g.rpb == 0) {
            // channel counts that are no multiple of 32: a plane that starts inside the tensor and ends outside it (or lies
            // outside altogether) arrives with zeros in the missing channels, which a plane-strided map cannot express
            mbar_expect_tx(&full_bar[s], STAGE);
            for (int pl = 0; pl < 4; ++pl) tma_load_2d(sa + pl * 4096, &tmA, (tile * 4 + pl) * 32, kb * 32, &full_bar[s]);
            for (int pl = 0; pl < BN / 32; ++pl) tma_load_2d(sb + pl * 4096, &tmB, n0 + pl * 32, kb * 32, &full_bar[s]);
          } else {
            // one box per 32-channel plane, so that the planes keep their 4096-byte pitch although a box has fewer than 32 rows
            mbar_expect_tx(&full_bar[s], (uint32_t)g.ppb * 128u * (4u + BN / 32u));
            for (int pl = 0; pl < 4; ++pl) tma_load_3d(sa + pl * 4096, &tmA, 0, kb * g.ppb, tile * 4 + pl, &full_bar[s]);
            for (int pl = 0; pl < BN / 32; ++pl) tma_load_4d(sb + pl * 4096, &tmB, 0, 0, kb * g.rpb, (n0 >> 5) + pl, &full_bar[s]);
          }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        for (int i = 0; i < nkb; ++i) {
          const int s = i % stages;
          if (!mbar_wait(&full_bar[s], (uint32_t)(i / stages) & 1u)) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); break; }
          tc_fence_after();
          const uint32_t sa = base + (uint32_t)s * STAGE, sb = sa + KC * A_BYTES;
          if (MODE != 1) {
            // descriptors differ only in their 14-bit start-address field (bytes >> 4): one add per MMA
            const uint64_t ad0 = make_desc(sa, 16, 1024) | LAYOUT_SW128, bd0 = make_desc(sb, 16, 1024) | LAYOUT_SW128;
#pragma unroll
            for (int u = 0; u < KC; ++u)
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                umma_tf32(tmem, ad0 + (uint64_t)((u * A_BYTES + kk * 32) >> 4), bd0 + (uint64_t)((u * B_BYTES + kk * 32) >> 4), IDESC,
                          (i | u | kk) ? 1u : 0u);
          } else {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t ad = make_desc(sa + kk * 1024, 4096, 512) | LAYOUT_SW128_BASE32;
              const uint64_t bd = make_desc(sb + kk * 1024, 4096, 512) | LAYOUT_SW128_BASE32;
              umma_tf32(tmem, ad, bd, IDESC, (i | kk) ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[s]);
        }
        umma_commit(&accum_bar);                           // arrives once every MMA issued above has completed
      }
      __syncwarp();
    } else {
      // ---- epilogue: TMEM lane quadrant (warp & 3) ----
      const bool done = mbar_wait(&accum_bar, 0);
      if (!done) { s_abort = 1; atomicExch(status, XB_TIMEOUT_MBAR); }
      tc_fence_after();
      const int q = warp & 3, half = (warp - 2) >> 2, row = q * 32 + lane;
      if (done && !s_abort) {
        if (MODE != 1) {
          long long m;
          bool ok;
          if (MODE == 0) {
            m = (long long)tile * g.mvalid + row;
            ok = row < g.mvalid && m < g.M;
            if (g.oQ && ok) {
              const int q = (int)(m % g.oQ); const long long t = m / g.oQ; const int pp = (int)(t % g.oP); const long long n = t / g.oP;
              m = (n * g.oH + 2 * pp) * g.oW + 2 * q;
            }
          } else {
            const int wt = tile % g.tiles_w, t2 = tile / g.tiles_w, ht = t2 % g.tiles_h, nt = t2 / g.tiles_h;
            const int wo = row % g.bw, t3 = row / g.bw, ho = t3 % g.bh, no = t3 / g.bh;
            const int w = wt * g.bw + wo, h = ht * g.bh + ho, n = nt * g.bn + no;
            ok = no < g.bn && w < g.W && h < g.H && n < g.NI;
            m = ((long long)n * g.H + h) * g.W + w;
          }
          // Thread = row after tcgen05.ld, but a row-per-thread store touches 32 lines per instruction.  So every warp
          // transposes 32 x 32 blocks through shared memory: afterwards eight lanes cover the 128 contiguous bytes of one
          // row, an instruction writes four full lines, and the batch-norm sums need two shuffles per column group.
          // (the pipeline stages are idle by now - every load has landed and every MMA has completed - and serve as the buffer)
          // The block is kept as 32 rows of eight 16-byte chunks, chunk j of row r at position j ^ (r & 7): the eight lanes
          // of a quarter-warp then hit all 32 banks both when a lane writes chunk j of ITS row and when eight lanes read the
          // eight chunks of ONE row, so the whole transpose is 8 + 8 conflict-free 16-byte accesses per lane.
          float4* tb4 = reinterpret_cast<float4*>(smem + (size_t)(warp - 2) * 32 * 32 * sizeof(float));
          s_rowoff[q][lane] = ok ? m * g.ldd : -1ll;
          __syncwarp();
          const int cq = (lane & 7) * 4, rsub = lane >> 3;
#pragma unroll 1
          for (int c0 = half * 32; c0 < BN; c0 += 64) {
            if (n0 + c0 >= g.N) break;                     // whole-warp condition
            {
              float v[32];                                 // one 32-column load: one wait instead of two
              tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
              for (int j = 0; j < 8; ++j) tb4[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
            __syncwarp();
            const int n = n0 + c0 + cq;                    // first of this lane's four columns
            const bool ncol = n < g.N;                     // (N is a multiple of 4)
            float b4[4] = {0.f, 0.f, 0.f, 0.f};
            if (bias && ncol && !((flags & G_SPLITK) && blockIdx.z)) { b4[0] = bias[n]; b4[1] = bias[n + 1]; b4[2] = bias[n + 2]; b4[3] = bias[n + 3]; }
            float sx[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + rsub;
              const long long off = s_rowoff[q][r];
              if (off >= 0 && ncol) {
                const float4 t4 = tb4[r * 8 + ((lane & 7) ^ (r & 7))];
                float x[4] = {t4.x + b4[0], t4.y + b4[1], t4.z + b4[2], t4.w + b4[3]};
                if (flags & G_RELU) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) x[k] = fmaxf(x[k], 0.f);
                }
                float4* o = reinterpret_cast<float4*>(D + off + n);
                if (flags & G_SPLITK) { red_add_v4(D + off + n, x[0], x[1], x[2], x[3]); continue; }
                if (flags & G_ACCUM) { const float4 old = *o; x[0] += old.x; x[1] += old.y; x[2] += old.z; x[3] += old.w; }
                *o = make_float4(x[0], x[1], x[2], x[3]);
                if (flags & G_BNBWD) {                     // x = final dy of a normalisation layer: its backward sums
                  const float4 bx = *reinterpret_cast<const float4*>(bn.x + off + n);
                  float4 by = make_float4(1.f, 1.f, 1.f, 1.f);
                  if (bn.relu) by = *reinterpret_cast<const float4*>(bn.y + off + n);
                  const float xv[4] = {bx.x, bx.y, bx.z, bx.w}, yv[4] = {by.x, by.y, by.z, by.w};
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    const float dz = yv[k] > 0.f ? x[k] : 0.f;
                    sx[k] += dz; sq[k] += dz * (xv[k] - bn.mean[n + k]) * bn.istd[n + k];
                  }
                } else {
#pragma unroll
                  for (int k = 0; k < 4; ++k) { sx[k] += x[k]; sq[k] += x[k] * x[k]; }
                }
              }
            }
            if (flags & (G_STATS | G_BNBWD)) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                sx[k] += __shfl_xor_sync(0xffffffffu, sx[k], 8);  sq[k] += __shfl_xor_sync(0xffffffffu, sq[k], 8);
                sx[k] += __shfl_xor_sync(0xffffffffu, sx[k], 16); sq[k] += __shfl_xor_sync(0xffffffffu, sq[k], 16);
              }
              if (lane < 8 && ncol) {
#pragma unroll
                for (int k = 0; k < 4; ++k) { atomicAdd(&s_red[c0 + cq + k], sx[k]); atomicAdd(&s_red[BN + c0 + cq + k], sq[k]); }
              }
            }
            __syncwarp();
          }
        } else {
          const int m = tile * 128 + row;
#pragma unroll 1
          for (int c0 = half * 16; c0 < BN; c0 += 32) {
            if (n0 + c0 >= g.N) break;
            float v[16];
            tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
            if (m < g.M) {
              float* orow = D + (long long)m * g.ldd + n0 + c0;
#pragma unroll
              for (int j = 0; j < 16; j += 4) if (n0 + c0 + j < g.N) red_add_v4(orow + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (MODE != 1 && (flags & (G_STATS | G_BNBWD)) && !s_abort) {
    for (int i = tid; i < BN; i += NTH) {
      const int n = n0 + i;
      if (n < g.N) { atomicAdd(&stats[n], s_red[i]); atomicAdd(&stats[g.N + n], s_red[BN + i]); }
    }
  }
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- host side ----------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rank-2 or rank-3 fp32 tensor map; strides[i] = bytes between consecutive indices of dimension i+1
int make_map(CUtensorMap* m, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -XB_BAD_ARG;
  const cuuint32_t ones[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -XB_BAD_ARG;
}

constexpr size_t kSmemLimit = 200 * 1024;
// Shared-memory budgets of the operand pipeline: `g_budget_many` when the grid has more CTAs than SMs, `g_budget_few`
// otherwise.  A CTA of a small grid used to take up to 200 KB for a deep pipeline; that kept every other replica's
// GEMM CTAs off its SM, and with four replicas per GPU the whole step paid for it: at 54 / 100 KB ResNet-32 (k = 4) went
// from 105.8 K to 117.0 K images/s, VGG-16 (k = 4) from 84.1 K to 87.7 K, ResNet-50 (k = 2) from 5.24 K to 5.28 K, and one
// replica alone lost nothing (47.7 K -> 47.9 K).
// (with output tiles capped at 128 columns a third 24 KB / a second 32 KB stage pays again for the wide layers: ResNet-50
// (k = 2) 5.41 K at 54 KB, 5.47 - 5.49 K at 72 - 80 KB, 5.29 K at 36 and at 108 KB; ResNet-32 is flat from 64 to 80 KB)
static size_t g_budget_many = 72 * 1024, g_budget_few = 100 * 1024;
inline size_t stage_bytes(int BN, int kc = 1) { return (size_t)kc * (A_BYTES + (size_t)BN * 128); }
// Pipeline depth: as deep as the reduction, within a shared-memory budget that still lets two CTAs share an SM when the
// grid has more CTAs than SMs (the second CTA's loads and MMAs then overlap the first one's epilogue).
inline int pick_stages(int steps, int BN, long long ctas, int kc = 1) {
  const size_t budget = ctas > 148 ? g_budget_many : g_budget_few;
  int s = steps < MAX_STAGES ? steps : MAX_STAGES;
  while (s > 2 && (size_t)s * stage_bytes(BN, kc) > budget) --s;
  return s;
}
// Reduction blocks per stage: as many as divide `blocks` (channel blocks per tap, or k-blocks of a plain GEMM) while at
// least two stages still fit; wide tiles keep one (their MMAs are long enough to hide the per-stage overhead).
inline int pick_kc(int blocks, int BN, long long ctas) {
  const size_t budget = ctas > 148 ? g_budget_many : g_budget_few;     // (same budget as pick_stages: keep two CTAs per SM)
  const int order[3] = {4, 2, 3};                        // (3 only where neither 4 nor 2 divides: nine taps of a 32-channel layer)
  for (int kc : order)
    if (blocks % kc == 0 && 2 * stage_bytes(BN, kc) <= budget && (BN <= 64 || kc <= 2)) return kc;
  return 1;
}

template <int BN, int MODE, int KC>
int launch_kc(const CUtensorMap& a, const CUtensorMap& b, float* D, const float* bias, float* stats, GemmArgs g, dim3 grid, int flags, int* status,
              cudaStream_t st, const XbBnFuse& bn) {
  size_t smem = (size_t)g.stages * stage_bytes(BN, KC);
  if (smem < (size_t)EPI_BYTES) smem = EPI_BYTES;          // the idle stages double as the epilogue's transpose blocks
  return (int)xb_launch(gemm_tma_kernel<BN, MODE, KC>, grid, dim3(gemm_threads(BN, MODE)), smem, st, a, b, D, bias, stats, g, flags, status, bn);
}
template <int BN, int MODE>
int launch(const CUtensorMap& a, const CUtensorMap& b, float* D, const float* bias, float* stats, GemmArgs g, dim3 grid, int flags, int* status,
           cudaStream_t st, const XbBnFuse& bn) {
  if (MODE != 1 && g.kc == 4) return launch_kc<BN, MODE == 1 ? 0 : MODE, (MODE == 1 || BN > 64) ? 1 : 4>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
  if (MODE != 1 && g.kc == 3) return launch_kc<BN, MODE == 1 ? 0 : MODE, (MODE == 1 || BN > 64) ? 1 : 3>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
  if (MODE != 1 && g.kc == 2) return launch_kc<BN, MODE == 1 ? 0 : MODE, MODE == 1 ? 1 : 2>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
  return launch_kc<BN, MODE, 1>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
}
template <int MODE>
int launch_bn(int BN, const CUtensorMap& a, const CUtensorMap& b, float* D, const float* bias, float* stats, GemmArgs g, dim3 grid, int flags,
              int* status, cudaStream_t st, const XbBnFuse& bn = XbBnFuse{}) {
  switch (BN) {
    case 32: return launch<32, MODE>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
    case 64: return launch<64, MODE>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
    case 128: return launch<128, MODE>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
    default: return launch<256, MODE>(a, b, D, bias, stats, g, grid, flags, status, st, bn);
  }
}
template <int BN, int MODE>
int configure() {
  int e;
  if ((e = (int)cudaFuncSetAttribute(gemm_tma_kernel<BN, MODE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  if (MODE != 1) {
    if ((e = (int)cudaFuncSetAttribute(gemm_tma_kernel<BN, MODE == 1 ? 0 : MODE, MODE == 1 ? 1 : 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
    if (BN <= 64 && (e = (int)cudaFuncSetAttribute(gemm_tma_kernel<BN, MODE == 1 ? 0 : MODE, (MODE == 1 || BN > 64) ? 1 : 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
    if (BN <= 64 && (e = (int)cudaFuncSetAttribute(gemm_tma_kernel<BN, MODE == 1 ? 0 : MODE, (MODE == 1 || BN > 64) ? 1 : 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit))) return e;
  }
  return 0;
}

static int g_tn_ctas = 111;                              // CTAs of a weight-gradient GEMM (output tiles x position slices)
inline bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool is_1x1(const XbConvGeom* g) { return g->R == 1 && g->S == 1 && g->ph == 0 && g->pw == 0 && g->sh == g->sw && (g->sh == 1 || g->sh == 2); }

}  // namespace

XB_API void xb_gemm_set_tn_ctas(int n) { g_tn_ctas = n > 0 ? n : 111; }
// widest output tile (TMEM columns per CTA) of the NT / CONV forms and of the TN form.  A 256-column tile lets only two
// CTAs share an SM's tensor memory, and these kernels hide one CTA's epilogue behind another CTA's main loop: ResNet-50
// (k = 2) 5.29 K -> 5.40 K images/s with 128 columns for NT / CONV, 5.16 K with 64; the TN form is indifferent (5.31 K).
static int g_max_bn_nt = 128, g_max_bn_tn = 256;
XB_API void xb_gemm_set_max_bn(int nt, int tn) {
  g_max_bn_nt = (nt == 32 || nt == 64 || nt == 128) ? nt : 256;
  g_max_bn_tn = (tn == 32 || tn == 64 || tn == 128) ? tn : 256;
}
static int g_split_k = 1;
XB_API void xb_gemm_set_split_k(int on) { g_split_k = on; }   // (A/B comparisons: 0 keeps every reduction inside one CTA)
XB_API void xb_gemm_set_smem_budgets(int many_kb, int few_kb) {
  g_budget_many = many_kb > 0 ? (size_t)(many_kb < 200 ? many_kb : 200) * 1024 : 54 * 1024;
  g_budget_few = few_kb > 0 ? (size_t)(few_kb < 200 ? few_kb : 200) * 1024 : 100 * 1024;
}
XB_API int xb_gemm_tma_init() {
  int e;
  if (!encode_fn()) return 0;                            // no driver entry point: the callers keep to the gather kernels
  if ((e = configure<32, 0>()) || (e = configure<64, 0>()) || (e = configure<128, 0>()) || (e = configure<256, 0>())) return e;
  if ((e = configure<32, 2>()) || (e = configure<64, 2>()) || (e = configure<128, 2>()) || (e = configure<256, 2>())) return e;
  if ((e = configure<32, 1>()) || (e = configure<64, 1>()) || (e = configure<128, 1>()) || (e = configure<256, 1>())) return e;
  return 0;
}

// which: 0 fprop, 1 dgrad, 2 wgrad; stride 1 or 2
XB_API int xb_conv1x1_tma_supported(const XbConvGeom* g, int which) {
  if (!encode_fn() || !is_1x1(g)) return 0;
  if (g->C % 4 || g->K % 4) return 0;
  if ((long long)g->N * g->H * g->W >= (1ll << 31)) return 0;
  if (which == 0) {
    if (g->sh == 1) return 1;
    return (g->H % 2 == 0 && g->W % 2 == 0 && g->Q <= 128) ? 1 : 0;
  }
  if (g->sh != 1 && (g->H % 2 || g->W % 2)) return 0;
  if (which == 1) return 1;
  // stride 1: any channel counts (multiples of 4); where they are no multiples of 32 the planes are loaded one by one
  // from rank-2 maps, the missing channels read the fill value (zero) and the epilogue only writes rows below K
  if (g->sh == 1) return 1;
  if (g->C % 32 || g->K % 32) return 0;
  return g->Q <= 32 ? 1 : 0;
}

// which 0: In = X (N,H,W,C), Wb = weights (K,C), Out = Y (N,P,Q,K).  which 1: In = dY (N,P,Q,K), Wb = transposed weights (C,K), Out = dX.
XB_API int xb_conv1x1_tma(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which, int flags,
                          int* status, cudaStream_t st, const XbBnFuse* bnf) {
  XbBnFuse bn{};
  if (bnf && bnf->sums) { bn = *bnf; stats = bnf->sums; flags = (flags & ~G_STATS) | G_BNBWD; }
  if (!aligned16p(In) || !aligned16p(Wb) || !aligned16p(Out) || !xb_conv1x1_tma_supported(cg, which)) return -XB_BAD_ARG;
  const int Kred = which == 0 ? cg->C : cg->K, Nout = which == 0 ? cg->K : cg->C;
  GemmArgs g{};
  CUtensorMap ta, tb;
  int tiles_m;
  if (cg->sh == 1 || which == 1) {
    // rows of the GEMM = consecutive pixels of In (for the data gradient of a stride-2 layer: of dY, the small image)
    const long long P = which == 1 ? (long long)cg->N * cg->P * cg->Q : (long long)cg->N * cg->H * cg->W;
    const cuuint64_t dims[3] = {(cuuint64_t)Kred, (cuuint64_t)P, 1};
    const cuuint64_t strides[2] = {(cuuint64_t)Kred * 4, (cuuint64_t)Kred * 4 * (cuuint64_t)P};
    const cuuint32_t box[3] = {32, 128, 1};
    if (make_map(&ta, In, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -XB_BAD_ARG;
    g.M = (int)P; g.mvalid = 128; g.c1_step = 128; g.c2_step = 0; g.a_bytes = (int)A_BYTES;
    tiles_m = (int)((P + 127) / 128);
    if (cg->sh == 2) {
      g.oP = cg->P; g.oQ = cg->Q; g.oH = cg->H; g.oW = cg->W;
      // pixels no output maps to receive no gradient: clear them unless the caller accumulates
      if (!(flags & G_ACCUM)) {
        cudaError_t e = cudaMemsetAsync(Out, 0, (size_t)cg->N * cg->H * cg->W * Nout * sizeof(float), st);
        if (e != cudaSuccess) return (int)e;
      }
    }
  } else {
    // stride 2: output pixel (n, p, q) reads input pixel (n, 2p, 2q); with H even, row n*H + 2p = 2 * (n*P + p)
    const int rows = cg->N * cg->P, bw = cg->Q, br = 128 / bw;
    const cuuint64_t dims[3] = {(cuuint64_t)Kred, (cuuint64_t)bw, (cuuint64_t)rows};
    const cuuint64_t strides[2] = {(cuuint64_t)Kred * 4 * 2, (cuuint64_t)Kred * 4 * 2 * (cuuint64_t)cg->W};
    const cuuint32_t box[3] = {32, (cuuint32_t)bw, (cuuint32_t)br};
    if (make_map(&ta, In, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -XB_BAD_ARG;
    g.M = rows * bw; g.mvalid = bw * br; g.c1_step = 0; g.c2_step = br; g.a_bytes = bw * br * 128;
    tiles_m = (rows + br - 1) / br;
  }
  int BN = Nout <= 32 ? 32 : Nout <= 64 ? 64 : Nout <= 128 ? 128 : 256;
  if (BN > g_max_bn_nt) BN = g_max_bn_nt;
  while (BN > 64 && (long long)tiles_m * ((Nout + BN - 1) / BN) < 148) BN >>= 1;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)Kred, (cuuint64_t)Nout};
    const cuuint64_t strides[1] = {(cuuint64_t)Kred * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)BN};
    if (make_map(&tb, Wb, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -XB_BAD_ARG;
  }
  g.N = Nout; g.kblocks = (Kred + 31) / 32; g.ldd = Nout;
  dim3 grid((unsigned)tiles_m, (unsigned)((Nout + BN - 1) / BN), 1);
  int steps = g.kblocks;
  // A product with few output tiles and a long reduction (an inner-product layer at batch size: 32 x 2048 x 1000 is 16
  // tiles) leaves most SMs idle while 16 CTAs stream the whole weight matrix: split the reduction over gridDim.z and let
  // every CTA add its partial tile.  Only where the epilogue is linear in the accumulator (no ReLU, no sums of the output).
  const long long tiles = (long long)grid.x * grid.y;
  if (g_split_k && cg->sh == 1 && !(flags & (G_RELU | G_STATS | G_BNBWD)) && tiles * 4 <= 148 && g.kblocks >= 8) {
    int splits = (int)((148 + tiles - 1) / tiles);
    if (splits > g.kblocks / 2) splits = g.kblocks / 2;
    g.kb_per_split = (g.kblocks + splits - 1) / splits;
    splits = (g.kblocks + g.kb_per_split - 1) / g.kb_per_split;
    if (splits > 1) {
      if (!(flags & G_ACCUM)) {
        cudaError_t e = cudaMemsetAsync(Out, 0, (size_t)g.M * Nout * sizeof(float), st);
        if (e != cudaSuccess) return (int)e;
      }
      flags |= G_SPLITK;
      grid.z = (unsigned)splits;
      steps = g.kb_per_split;
    } else {
      g.kb_per_split = 0;
    }
  }
  g.stages = pick_stages(steps, BN, tiles * grid.z);
  return launch_bn<0>(BN, ta, tb, Out, bias, stats, g, grid, flags, status, st, bn);
}

// dW (K,C) += dY^T X over all positions; dW must hold the value to accumulate onto (normally zero).
XB_API int xb_conv1x1_wgrad_tma(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st) {
  if (!aligned16p(dY) || !aligned16p(X) || !aligned16p(dW) || !xb_conv1x1_tma_supported(cg, 2)) return -XB_BAD_ARG;
  const long long P = (long long)cg->N * cg->P * cg->Q;   // positions of dY
  int BN = cg->C <= 32 ? 32 : cg->C <= 64 ? 64 : cg->C <= 128 ? 128 : 256;
  if (BN > g_max_bn_tn) BN = g_max_bn_tn;
  const int rpb = cg->sh == 1 ? 0 : (32 / cg->Q < cg->N * cg->P ? 32 / cg->Q : cg->N * cg->P), ppb = rpb * cg->Q;
  const int planes2d = cg->sh == 1 && (cg->C % 32 || (cg->K % 32 && cg->K > 32));
  CUtensorMap ta, tb;
  if (planes2d) {
    const cuuint64_t da[2] = {(cuuint64_t)cg->K, (cuuint64_t)P}, sa[1] = {(cuuint64_t)cg->K * 4};
    const cuuint64_t db[2] = {(cuuint64_t)cg->C, (cuuint64_t)P}, sb[1] = {(cuuint64_t)cg->C * 4};
    const cuuint32_t box[2] = {32, 32};
    if (make_map(&ta, dY, 2, da, sa, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -XB_BAD_ARG;
    if (make_map(&tb, X, 2, db, sb, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -XB_BAD_ARG;
  } else {
    const cuuint64_t dims[3] = {(cuuint64_t)(cg->K < 32 ? cg->K : 32), (cuuint64_t)P, (cuuint64_t)((cg->K + 31) / 32)};
    const cuuint64_t strides[2] = {(cuuint64_t)cg->K * 4, 128};
    const cuuint32_t box[3] = {32, (cuuint32_t)(rpb ? ppb : 32), (cuuint32_t)(rpb ? 1 : 4)};
    if (make_map(&ta, dY, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -XB_BAD_ARG;
  }
  if (planes2d) {
  } else if (rpb == 0) {
    const cuuint64_t dims[3] = {32, (cuuint64_t)P, (cuuint64_t)(cg->C / 32)};
    const cuuint64_t strides[2] = {(cuuint64_t)cg->C * 4, 128};
    const cuuint32_t box[3] = {32, 32, (cuuint32_t)(BN / 32)};
    if (make_map(&tb, X, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -XB_BAD_ARG;
  } else {
    // every second pixel of every second row: (channel in plane, q, n*P + p, plane)
    const cuuint64_t dims[4] = {32, (cuuint64_t)cg->Q, (cuuint64_t)cg->N * cg->P, (cuuint64_t)(cg->C / 32)};
    const cuuint64_t strides[3] = {(cuuint64_t)cg->C * 4 * 2, (cuuint64_t)cg->C * 4 * 2 * cg->W, 128};
    const cuuint32_t box[4] = {32, (cuuint32_t)cg->Q, (cuuint32_t)rpb, 1};
    if (make_map(&tb, X, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return -XB_BAD_ARG;
  }
  GemmArgs g{};
  g.M = cg->K; g.N = cg->C; g.ldd = cg->C; g.rpb = rpb; g.ppb = ppb; g.kc = 1; g.planes2d = planes2d;
  g.kblocks = rpb ? (cg->N * cg->P + rpb - 1) / rpb : (int)((P + 31) / 32);
  const int tiles = ((cg->K + 127) / 128) * ((cg->C + BN - 1) / BN);
  int splits = (g_tn_ctas + tiles - 1) / tiles;
  if (splits > g.kblocks) splits = g.kblocks;
  g.kb_per_split = (g.kblocks + splits - 1) / splits;
  splits = (g.kblocks + g.kb_per_split - 1) / g.kb_per_split;
  dim3 grid((unsigned)((cg->K + 127) / 128), (unsigned)((cg->C + BN - 1) / BN), (unsigned)splits);
  g.stages = pick_stages(g.kb_per_split, BN, (long long)grid.x * grid.y * grid.z);
  return launch_bn<1>(BN, ta, tb, dW, nullptr, nullptr, g, grid, 0, status, st);
}

// which: 0 fprop (C % 32 == 0), 1 dgrad (K % 32 == 0).  R x S, stride 1, output extent = input extent.
XB_API int xb_conv_tma_supported(const XbConvGeom* g, int which) {
  if (!encode_fn()) return 0;
  if (g->sh != 1 || g->sw != 1 || g->P != g->H || g->Q != g->W) return 0;
  if (2 * g->ph != g->R - 1 || 2 * g->pw != g->S - 1) return 0;
  const int Kred = which == 0 ? g->C : g->K, Nout = which == 0 ? g->K : g->C;
  if (which > 1 || Kred % 32 || Nout % 4) return 0;
  return 1;
}

// which 0: In = X, Wb = weights (K,R,S,C), Out = Y.  which 1: In = dY, Wb = transposed weights (C,R,S,K), Out = dX.
XB_API int xb_conv_tma(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which, int flags,
                       int* status, cudaStream_t st, const XbBnFuse* bnf) {
  XbBnFuse bn{};
  if (bnf && bnf->sums) { bn = *bnf; stats = bnf->sums; flags = (flags & ~G_STATS) | G_BNBWD; }
  if (!aligned16p(In) || !aligned16p(Wb) || !aligned16p(Out) || !xb_conv_tma_supported(cg, which)) return -XB_BAD_ARG;
  const int Kred = which == 0 ? cg->C : cg->K, Nout = which == 0 ? cg->K : cg->C;
  GemmArgs g{};
  g.H = cg->H; g.W = cg->W; g.NI = cg->N; g.R = cg->R; g.S = cg->S; g.ph = cg->ph; g.pw = cg->pw;
  g.bw = cg->W < 128 ? cg->W : 128;
  g.bh = 128 / g.bw < cg->H ? 128 / g.bw : cg->H;
  if (g.bh < 1) g.bh = 1;
  g.bn = 128 / (g.bw * g.bh) < cg->N ? 128 / (g.bw * g.bh) : cg->N;
  if (g.bn < 1) g.bn = 1;
  g.tiles_w = (cg->W + g.bw - 1) / g.bw; g.tiles_h = (cg->H + g.bh - 1) / g.bh;
  const int tiles_m = g.tiles_w * g.tiles_h * ((cg->N + g.bn - 1) / g.bn);
  g.c32 = Kred / 32; g.mirrored = which; g.krow = Kred;
  g.a_bytes = g.bw * g.bh * g.bn * 128;
  g.M = cg->N * cg->H * cg->W; g.N = Nout; g.ldd = Nout;
  CUtensorMap ta, tb;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)Kred, (cuuint64_t)cg->W, (cuuint64_t)cg->H, (cuuint64_t)cg->N};
    const cuuint64_t strides[3] = {(cuuint64_t)Kred * 4, (cuuint64_t)Kred * 4 * cg->W, (cuuint64_t)Kred * 4 * cg->W * cg->H};
    const cuuint32_t box[4] = {32, (cuuint32_t)g.bw, (cuuint32_t)g.bh, (cuuint32_t)g.bn};
    if (make_map(&ta, In, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -XB_BAD_ARG;
  }
  int BN = Nout <= 32 ? 32 : Nout <= 64 ? 64 : Nout <= 128 ? 128 : 256;
  if (BN > g_max_bn_nt) BN = g_max_bn_nt;
  while (BN > 32 && (long long)tiles_m * ((Nout + BN - 1) / BN) < 120) BN >>= 1;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)cg->R * cg->S * Kred, (cuuint64_t)Nout};
    const cuuint64_t strides[1] = {(cuuint64_t)cg->R * cg->S * Kred * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)BN};
    if (make_map(&tb, Wb, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -XB_BAD_ARG;
  }
  dim3 grid((unsigned)tiles_m, (unsigned)((Nout + BN - 1) / BN), 1);
  g.kc = pick_kc(cg->R * cg->S * g.c32, BN, (long long)grid.x * grid.y);
  g.kblocks = cg->R * cg->S * g.c32 / g.kc;              // pipeline steps: (tap, group of kc channel blocks)
  g.stages = pick_stages(g.kblocks, BN, (long long)grid.x * grid.y, g.kc);
  return launch_bn<2>(BN, ta, tb, Out, bias, stats, g, grid, flags, status, st, bn);
}
