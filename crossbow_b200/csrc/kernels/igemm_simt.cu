// Implicit-GEMM convolution / inner product on CUDA cores (fp32 FMA), channels-last.
//
// Three products share one register-tiled inner loop:
//   fprop : Y[(n,p,q), k]    = sum_{r,s,c} X[n, p*sh-ph+r, q*sw-pw+s, c] * W[k, r, s, c]         (+bias, ReLU, BN partial sums)
//   dgrad : dX[(n,h,w), c]   = sum_{r,s,k} dY[n, (h+ph-r)/sh, (w+pw-s)/sw, k] * Wt[c, r, s, k]    (Wt = weights with K and C swapped)
//   wgrad : dW[k, (r,s,c)]   = sum_{n,p,q} dY[(n,p,q), k] * X[n, p*sh-ph+r, q*sw-pw+s, c]         (split over pixels, atomic accumulate)
//
// This is the exact-fp32 path: it serves shapes the tensor-core kernels do not cover (reduction extents that are
// not a multiple of 4, e.g. the 3-channel first layer) and is the in-library cross-check for them.
// Replaces cudnnConvolutionForward/BackwardData/BackwardFilter + cublasSgemm call sites of
// clib-multigpu/kernels/cudnnconv.cu:96-124, cudnnconvgradient.cu:72-169, innerproduct.cu:133-169,
// innerproductgradient.cu:88-152.
#include "common.cuh"

namespace {

constexpr int BK = 16;

// Gather problem: rows of the GEMM are output positions, the reduction runs over (r, s, c).
struct GatherProblem {
  int M;            // rows = N*OH*OW
  int OH, OW;       // output grid
  int IH, IW, CR;   // source grid and reduction channels
  int NG;           // GEMM N (output channels)
  int R, S;
  int sh, sw, ph, pw;
  int transposed;   // 0: iy = oy*sh-ph+r ; 1: iy = (oy+ph-r)/sh when divisible
  int KG;           // R*S*CR
};

__device__ __forceinline__ bool src_coord(const GatherProblem& g, int oy, int ox, int r, int s, int& iy, int& ix) {
  if (!g.transposed) {
    iy = oy * g.sh - g.ph + r;
    ix = ox * g.sw - g.pw + s;
  } else {
    int ty = oy + g.ph - r, tx = ox + g.pw - s;
    if (ty < 0 || tx < 0) return false;
    if (g.sh > 1) { if (ty % g.sh) return false; ty /= g.sh; }
    if (g.sw > 1) { if (tx % g.sw) return false; tx /= g.sw; }
    iy = ty; ix = tx;
  }
  return iy >= 0 && iy < g.IH && ix >= 0 && ix < g.IW;
}

template <int BM, int BN, int TM, int TN>
__device__ __forceinline__ void tile_fma(const float (*As)[BM + 4], const float (*Bs)[BN + 4], float (&acc)[TM][TN], int ty, int tx) {
#pragma unroll
  for (int kk = 0; kk < BK; ++kk) {
    float a[TM], b[TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
    for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// flags
constexpr int F_RELU = 1, F_ACCUM = 2, F_STATS = 4;

template <int BM, int BN, int TM, int TN, int VEC>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
igemm_gather_kernel(const float* __restrict__ A, const float* __restrict__ Bw, const float* __restrict__ bias,
                    float* __restrict__ Out, float* __restrict__ stats, GatherProblem g, int flags) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int KV = BK / VEC;                       // vectors per row per k-tile
  constexpr int LA = (BM * KV + NT - 1) / NT;        // A vectors per thread
  constexpr int LB = (BN * KV + NT - 1) / NT;
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;

  // fixed per-thread row bookkeeping for A
  int a_row[LA], a_oy[LA], a_ox[LA], a_kv[LA];
  long long a_base[LA];
#pragma unroll
  for (int i = 0; i < LA; ++i) {
    int v = tid + i * NT;
    int row = v / KV;
    a_kv[i] = v % KV;
    a_row[i] = (v < BM * KV) ? row : -1;
    int m = m0 + row;
    if (a_row[i] >= 0 && m < g.M) {
      int ox = m % g.OW; int t = m / g.OW; int oy = t % g.OH; int n = t / g.OH;
      a_oy[i] = oy; a_ox[i] = ox; a_base[i] = (long long)n * g.IH * g.IW * g.CR;
    } else {
      a_oy[i] = 0; a_ox[i] = 0; a_base[i] = -1;
    }
  }

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  float ra[LA][VEC], rb[LB][VEC];
  const int ktiles = (g.KG + BK - 1) / BK;

  auto load_tile = [&](int kt) {
    const int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < LA; ++i) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) ra[i][e] = 0.f;
      if (a_row[i] < 0 || a_base[i] < 0) continue;
      int k = k0 + a_kv[i] * VEC;
      if (VEC == 4) {
        if (k < g.KG) {
          int c = k % g.CR; int rs = k / g.CR; int s = rs % g.S; int r = rs / g.S;
          int iy, ix;
          if (src_coord(g, a_oy[i], a_ox[i], r, s, iy, ix)) {
            const float4 v = *reinterpret_cast<const float4*>(A + a_base[i] + ((long long)iy * g.IW + ix) * g.CR + c);
            ra[i][0] = v.x; ra[i][1 % VEC] = v.y; ra[i][2 % VEC] = v.z; ra[i][3 % VEC] = v.w;
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          int kk = k + e;
          if (kk < g.KG) {
            int c = kk % g.CR; int rs = kk / g.CR; int s = rs % g.S; int r = rs / g.S;
            int iy, ix;
            if (src_coord(g, a_oy[i], a_ox[i], r, s, iy, ix))
              ra[i][e] = A[a_base[i] + ((long long)iy * g.IW + ix) * g.CR + c];
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) rb[i][e] = 0.f;
      int v = tid + i * NT;
      if (v >= BN * KV) continue;
      int row = v / KV, kv = v % KV;
      int n = n0 + row, k = k0 + kv * VEC;
      if (n >= g.NG) continue;
      if (VEC == 4) {
        if (k < g.KG) {
          const float4 w = *reinterpret_cast<const float4*>(Bw + (long long)n * g.KG + k);
          rb[i][0] = w.x; rb[i][1 % VEC] = w.y; rb[i][2 % VEC] = w.z; rb[i][3 % VEC] = w.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          if (k + e < g.KG) rb[i][e] = Bw[(long long)n * g.KG + k + e];
      }
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int i = 0; i < LA; ++i) {
      if (a_row[i] < 0) continue;
#pragma unroll
      for (int e = 0; e < VEC; ++e) As[a_kv[i] * VEC + e][a_row[i]] = ra[i][e];
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
      int v = tid + i * NT;
      if (v >= BN * KV) continue;
      int row = v / KV, kv = v % KV;
#pragma unroll
      for (int e = 0; e < VEC; ++e) Bs[kv * VEC + e][row] = rb[i][e];
    }
  };

  load_tile(0);
  store_tile();
  __syncthreads();
  for (int kt = 0; kt < ktiles; ++kt) {
    if (kt + 1 < ktiles) load_tile(kt + 1);
    tile_fma<BM, BN, TM, TN>(As, Bs, acc, ty, tx);
    __syncthreads();
    if (kt + 1 < ktiles) {
      store_tile();
      __syncthreads();
    }
  }

  // epilogue
  float csum[TN], csq[TN];
#pragma unroll
  for (int j = 0; j < TN; ++j) { csum[j] = 0.f; csq[j] = 0.f; }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + ty * TM + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int n = n0 + tx * TN + j;
      if (n >= g.NG) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      if (flags & F_RELU) v = fmaxf(v, 0.f);
      float* o = Out + (long long)m * g.NG + n;
      if (flags & F_ACCUM) v += *o;
      *o = v;
      csum[j] += v; csq[j] += v * v;
    }
  }
  if (flags & F_STATS) {
    // per-channel partial sums of this tile: reduce over ty through shared memory, then one atomic per channel
    __syncthreads();
    float* red = &As[0][0];            // reuse: needs 2*BN floats per ty-group; do it with atomics in smem
    for (int i = tid; i < 2 * BN; i += NT) red[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      atomicAdd(&red[tx * TN + j], csum[j]);
      atomicAdd(&red[BN + tx * TN + j], csq[j]);
    }
    __syncthreads();
    for (int i = tid; i < BN; i += NT) {
      int n = n0 + i;
      if (n < g.NG) {
        atomicAdd(&stats[n], red[i]);
        atomicAdd(&stats[g.NG + n], red[BN + i]);
      }
    }
  }
}

// ---- wgrad ---------------------------------------------------------------------------------
struct WgradProblem {
  int NPIX;          // N*P*Q (reduction)
  int P, Q, H, W, C, K, R, S, sh, sw, ph, pw;
  int NG;            // R*S*C
  int pix_per_split;
};

template <int BM, int BN, int TM, int TN, int VEC>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
igemm_wgrad_kernel(const float* __restrict__ dY, const float* __restrict__ X, float* __restrict__ dW, WgradProblem g) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int MV = BM / VEC, NV = BN / VEC;
  constexpr int LA = (BK * MV + NT - 1) / NT;
  constexpr int LB = (BK * NV + NT - 1) / NT;
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int pix0 = blockIdx.z * g.pix_per_split;
  const int pix1 = min(g.NPIX, pix0 + g.pix_per_split);

  // B columns are fixed per thread: n -> (r, s, c)
  int b_kk[LB], b_nv[LB], b_r[LB], b_s[LB], b_c[LB];
#pragma unroll
  for (int i = 0; i < LB; ++i) {
    int v = tid + i * NT;
    b_kk[i] = (v < BK * NV) ? v / NV : -1;
    b_nv[i] = v % NV;
    int n = n0 + b_nv[i] * VEC;
    if (n < g.NG) { b_c[i] = n % g.C; int rs = n / g.C; b_s[i] = rs % g.S; b_r[i] = rs / g.S; }
    else { b_c[i] = -1; b_s[i] = 0; b_r[i] = 0; }
  }

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  float ra[LA][VEC], rb[LB][VEC];

  auto load_tile = [&](int p0) {
#pragma unroll
    for (int i = 0; i < LA; ++i) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) ra[i][e] = 0.f;
      int v = tid + i * NT;
      if (v >= BK * MV) continue;
      int kk = v / MV, mv = v % MV;
      int pix = p0 + kk, m = m0 + mv * VEC;
      if (pix >= pix1) continue;
      if (VEC == 4) {
        if (m < g.K) {
          const float4 t = *reinterpret_cast<const float4*>(dY + (long long)pix * g.K + m);
          ra[i][0] = t.x; ra[i][1 % VEC] = t.y; ra[i][2 % VEC] = t.z; ra[i][3 % VEC] = t.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) if (m + e < g.K) ra[i][e] = dY[(long long)pix * g.K + m + e];
      }
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) rb[i][e] = 0.f;
      if (b_kk[i] < 0) continue;
      int pix = p0 + b_kk[i];
      if (pix >= pix1) continue;
      int q = pix % g.Q; int t = pix / g.Q; int p = t % g.P; int n = t / g.P;
      if (VEC == 4) {
        if (b_c[i] < 0) continue;
        int iy = p * g.sh - g.ph + b_r[i], ix = q * g.sw - g.pw + b_s[i];
        if (iy < 0 || iy >= g.H || ix < 0 || ix >= g.W) continue;
        const float4 t4 = *reinterpret_cast<const float4*>(X + (((long long)n * g.H + iy) * g.W + ix) * g.C + b_c[i]);
        rb[i][0] = t4.x; rb[i][1 % VEC] = t4.y; rb[i][2 % VEC] = t4.z; rb[i][3 % VEC] = t4.w;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          int nn = n0 + b_nv[i] * VEC + e;
          if (nn >= g.NG) continue;
          int c = nn % g.C; int rs = nn / g.C; int s = rs % g.S; int r = rs / g.S;
          int iy = p * g.sh - g.ph + r, ix = q * g.sw - g.pw + s;
          if (iy < 0 || iy >= g.H || ix < 0 || ix >= g.W) continue;
          rb[i][e] = X[(((long long)n * g.H + iy) * g.W + ix) * g.C + c];
        }
      }
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int i = 0; i < LA; ++i) {
      int v = tid + i * NT;
      if (v >= BK * MV) continue;
      int kk = v / MV, mv = v % MV;
#pragma unroll
      for (int e = 0; e < VEC; ++e) As[kk][mv * VEC + e] = ra[i][e];
    }
#pragma unroll
    for (int i = 0; i < LB; ++i) {
      if (b_kk[i] < 0) continue;
#pragma unroll
      for (int e = 0; e < VEC; ++e) Bs[b_kk[i]][b_nv[i] * VEC + e] = rb[i][e];
    }
  };

  if (pix0 < pix1) {
    load_tile(pix0);
    store_tile();
    __syncthreads();
    for (int p0 = pix0; p0 < pix1; p0 += BK) {
      bool more = p0 + BK < pix1;
      if (more) load_tile(p0 + BK);
      tile_fma<BM, BN, TM, TN>(As, Bs, acc, ty, tx);
      __syncthreads();
      if (more) { store_tile(); __syncthreads(); }
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int m = m0 + ty * TM + i;
    if (m >= g.K) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int n = n0 + tx * TN + j;
      if (n >= g.NG) continue;
      atomicAdd(dW + (long long)m * g.NG + n, acc[i][j]);
    }
  }
}

template <int BM, int BN, int TM, int TN>
int launch_gather(const float* A, const float* Bw, const float* bias, float* Out, float* stats, const GatherProblem& g,
                  int flags, bool vec4, cudaStream_t st) {
  dim3 grid(xb_ceil_div(g.M, BM), xb_ceil_div(g.NG, BN));
  constexpr int NT = (BM / TM) * (BN / TN);
  if (vec4) igemm_gather_kernel<BM, BN, TM, TN, 4><<<grid, NT, 0, st>>>(A, Bw, bias, Out, stats, g, flags);
  else      igemm_gather_kernel<BM, BN, TM, TN, 1><<<grid, NT, 0, st>>>(A, Bw, bias, Out, stats, g, flags);
  return (int)cudaGetLastError();
}

int dispatch_gather(const float* A, const float* Bw, const float* bias, float* Out, float* stats, const GatherProblem& g,
                    int flags, cudaStream_t st) {
  bool vec4 = (g.CR % 4 == 0) && ((((uintptr_t)A) | ((uintptr_t)Bw)) % 16 == 0);
  // tile choice: narrow N tiles for few output channels; smaller M tiles when the grid would not fill the GPU
  long long rows128 = xb_ceil_div(g.M, 128);
  if (g.NG <= 16) {
    if (rows128 >= 148) return launch_gather<128, 16, 8, 2>(A, Bw, bias, Out, stats, g, flags, vec4, st);
    return launch_gather<64, 16, 4, 2>(A, Bw, bias, Out, stats, g, flags, vec4, st);
  }
  if (g.NG <= 32) {
    if (rows128 >= 148) return launch_gather<128, 32, 8, 4>(A, Bw, bias, Out, stats, g, flags, vec4, st);
    return launch_gather<64, 32, 4, 4>(A, Bw, bias, Out, stats, g, flags, vec4, st);
  }
  long long tiles = rows128 * xb_ceil_div(g.NG, 64);
  if (tiles >= 148) return launch_gather<128, 64, 8, 8>(A, Bw, bias, Out, stats, g, flags, vec4, st);
  if ((long long)xb_ceil_div(g.M, 64) * xb_ceil_div(g.NG, 64) >= 96)
    return launch_gather<64, 64, 4, 8>(A, Bw, bias, Out, stats, g, flags, vec4, st);
  return launch_gather<32, 32, 2, 4>(A, Bw, bias, Out, stats, g, flags, vec4, st);
}

}  // namespace

// flags: bit0 ReLU, bit1 accumulate into Out, bit2 accumulate per-channel sum / sum-of-squares into stats[2*K]
XB_API int xb_conv_fprop_simt(const float* X, const float* W, const float* bias, float* Y, float* stats, const XbConvGeom* cg,
                              int flags, cudaStream_t st) {
  GatherProblem g;
  g.M = cg->N * cg->P * cg->Q; g.OH = cg->P; g.OW = cg->Q; g.IH = cg->H; g.IW = cg->W; g.CR = cg->C; g.NG = cg->K;
  g.R = cg->R; g.S = cg->S; g.sh = cg->sh; g.sw = cg->sw; g.ph = cg->ph; g.pw = cg->pw; g.transposed = 0;
  g.KG = cg->R * cg->S * cg->C;
  return dispatch_gather(X, W, bias, Y, stats, g, flags, st);
}

// Wt is the (C,R,S,K) transposed copy of the weights (see xb_transpose_weights).
XB_API int xb_conv_dgrad_simt(const float* dY, const float* Wt, float* dX, const XbConvGeom* cg, int accumulate, cudaStream_t st) {
  GatherProblem g;
  g.M = cg->N * cg->H * cg->W; g.OH = cg->H; g.OW = cg->W; g.IH = cg->P; g.IW = cg->Q; g.CR = cg->K; g.NG = cg->C;
  g.R = cg->R; g.S = cg->S; g.sh = cg->sh; g.sw = cg->sw; g.ph = cg->ph; g.pw = cg->pw; g.transposed = 1;
  g.KG = cg->R * cg->S * cg->K;
  return dispatch_gather(dY, Wt, nullptr, dX, nullptr, g, accumulate ? F_ACCUM : 0, st);
}

// dW must be zero (or hold a value to accumulate onto) before the call.
XB_API int xb_conv_wgrad_simt(const float* dY, const float* X, float* dW, const XbConvGeom* cg, cudaStream_t st) {
  WgradProblem g;
  g.NPIX = cg->N * cg->P * cg->Q; g.P = cg->P; g.Q = cg->Q; g.H = cg->H; g.W = cg->W; g.C = cg->C; g.K = cg->K;
  g.R = cg->R; g.S = cg->S; g.sh = cg->sh; g.sw = cg->sw; g.ph = cg->ph; g.pw = cg->pw; g.NG = cg->R * cg->S * cg->C;
  bool vec4 = (cg->C % 4 == 0) && (cg->K % 4 == 0) && ((((uintptr_t)dY) | ((uintptr_t)X)) % 16 == 0);
  constexpr int BM = 64, BN = 64, TM = 4, TN = 8;
  constexpr int BMs = 16, BNs = 64, TMs = 2, TNs = 4;
  bool small = cg->K <= 16;
  int tiles = small ? xb_ceil_div(g.NG, BNs) * xb_ceil_div(g.K, BMs) : xb_ceil_div(g.NG, BN) * xb_ceil_div(g.K, BM);
  int max_splits = xb_ceil_div(g.NPIX, 4 * BK);
  int splits = xb_ceil_div(2 * 148, tiles);
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  g.pix_per_split = xb_ceil_div(xb_ceil_div(g.NPIX, splits), BK) * BK;
  splits = xb_ceil_div(g.NPIX, g.pix_per_split);
  if (small) {
    dim3 grid(xb_ceil_div(g.NG, BNs), xb_ceil_div(g.K, BMs), splits);
    constexpr int NT = (BMs / TMs) * (BNs / TNs);
    if (vec4) igemm_wgrad_kernel<BMs, BNs, TMs, TNs, 4><<<grid, NT, 0, st>>>(dY, X, dW, g);
    else      igemm_wgrad_kernel<BMs, BNs, TMs, TNs, 1><<<grid, NT, 0, st>>>(dY, X, dW, g);
  } else {
    dim3 grid(xb_ceil_div(g.NG, BN), xb_ceil_div(g.K, BM), splits);
    constexpr int NT = (BM / TM) * (BN / TN);
    if (vec4) igemm_wgrad_kernel<BM, BN, TM, TN, 4><<<grid, NT, 0, st>>>(dY, X, dW, g);
    else      igemm_wgrad_kernel<BM, BN, TM, TN, 1><<<grid, NT, 0, st>>>(dY, X, dW, g);
  }
  return (int)cudaGetLastError();
}

// ---- batched weight transpose (K,R,S,C) -> (C,R,S,K) for every convolution of a model, ONE launch -------
struct XbTransposeDesc { long long src_off, dst_off; int K, RS, C; int first_block; };

// One block = one 32 (k) x 32 (c) tile of one filter tap, moved through shared memory so that both the loads (along c) and
// the stores (along k) are coalesced.
__global__ void __launch_bounds__(256) transpose_weights_kernel(const float* __restrict__ w, float* __restrict__ wt, const XbTransposeDesc* __restrict__ d, int nd) {
  __shared__ float tile[32][33];
  // find the descriptor this block belongs to (descriptors are sorted by first_block)
  int lo = 0, hi = nd - 1;
  while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (d[mid].first_block <= (int)blockIdx.x) lo = mid; else hi = mid - 1; }
  const XbTransposeDesc e = d[lo];
  const int kt = (e.K + 31) >> 5, ct = (e.C + 31) >> 5;
  int b = (int)blockIdx.x - e.first_block;
  const int c0 = (b % ct) << 5; b /= ct;
  const int k0 = (b % kt) << 5; const int rs = b / kt;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const float* src = w + e.src_off;
  float* dst = wt + e.dst_off;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int k = k0 + ty + j, c = c0 + tx;
    tile[ty + j][tx] = (k < e.K && c < e.C) ? src[((long long)k * e.RS + rs) * e.C + c] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int c = c0 + ty + j, k = k0 + tx;
    if (c < e.C && k < e.K) dst[((long long)c * e.RS + rs) * e.K + k] = tile[tx][ty + j];
  }
}

// blocks the kernel above needs for one (K, RS, C) filter bank - the caller lays out first_block with this
XB_API int xb_transpose_blocks(int K, int RS, int C) { return ((K + 31) / 32) * ((C + 31) / 32) * RS; }

XB_API int xb_transpose_weights(const float* w, float* wt, const XbTransposeDesc* descs_dev, int nd, int total_blocks, cudaStream_t st) {
  if (nd == 0) return 0;
  transpose_weights_kernel<<<total_blocks, 256, 0, st>>>(w, wt, descs_dev, nd);
  return (int)cudaGetLastError();
}
