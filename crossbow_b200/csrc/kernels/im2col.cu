// Convolutions that no direct tensor-core kernel covers (3-channel first layers, strided R x S filters) as
// "lower to a matrix, then GEMM": a gather kernel writes the patch matrix A[m][(r,s,c)] with the reduction padded to a
// multiple of 32 floats, and the TMA-fed tcgen05 GEMM does the arithmetic -
//   forward          Y  = A  W_p^T      (W_p = filter bank with padded rows)
//   weight gradient  dW = dY^T A        (accumulated into a padded scratch, then folded into dW)
// The patch matrix lives in a caller-provided scratch region: one region per learner serves all such layers, because a
// learner's operators run in stream order.
#include "common.cuh"

XB_API int xb_conv1x1_tma_supported(const XbConvGeom* g, int which);
XB_API int xb_conv1x1_tma(const float* In, const float* Wb, const float* bias, float* Out, float* stats, const XbConvGeom* cg, int which, int flags,
                          int* status, cudaStream_t st, const XbBnFuse* bnf);
XB_API int xb_conv1x1_wgrad_tma(const float* dY, const float* X, float* dW, const XbConvGeom* cg, int* status, cudaStream_t st);

namespace {

inline int padded_k(const XbConvGeom* g) { return (g->R * g->S * g->C + 31) / 32 * 32; }
inline size_t align256(size_t b) { return (b + 255) / 256 * 256; }

// A thread keeps four consecutive reduction indices (their tap / channel decomposition is computed once) and walks the
// output positions of its block's slice; the Kp/4 threads of a position write one contiguous row of the patch matrix.
__global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ X, float* __restrict__ A, XbConvGeom g, int Kp, long long M, int rows_per_block) {
  const int k4n = Kp >> 2;
  const int per = 256 / k4n;                               // positions handled side by side by one block (>= 1 for Kp <= 1024)
  const int lane_k = threadIdx.x % k4n, sub = threadIdx.x / k4n;
  if (sub >= per) return;
  const int k0 = lane_k * 4, KR = g.R * g.S * g.C;
  int rr[4], ss[4], cc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = k0 + j, tap = k / g.C;
    cc[j] = k - tap * g.C; rr[j] = tap / g.S; ss[j] = tap - rr[j] * g.S;
    if (k >= KR) rr[j] = -1000000;                         // padding column: always out of range -> zero
  }
  const bool vec = (g.C & 3) == 0;
  const long long m0 = (long long)blockIdx.x * rows_per_block, m1 = m0 + rows_per_block < M ? m0 + rows_per_block : M;
  for (long long m = m0 + sub; m < m1; m += per) {
    const int q = (int)(m % g.Q); const long long t = m / g.Q; const int p = (int)(t % g.P); const int n = (int)(t / g.P);
    const int hb = p * g.sh - g.ph, wb = q * g.sw - g.pw;
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec) {                                             // four channels of one tap: one 16-byte load
      const int h = hb + rr[0], w = wb + ss[0];
      if (h >= 0 && h < g.H && w >= 0 && w < g.W) out = *reinterpret_cast<const float4*>(X + (((long long)n * g.H + h) * g.W + w) * g.C + cc[0]);
    } else {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int h = hb + rr[j], w = wb + ss[j];
        v[j] = (h >= 0 && h < g.H && w >= 0 && w < g.W) ? __ldg(X + (((long long)n * g.H + h) * g.W + w) * g.C + cc[j]) : 0.f;
      }
      out = make_float4(v[0], v[1], v[2], v[3]);
    }
    *reinterpret_cast<float4*>(A + m * Kp + k0) = out;
  }
}

// dst[row][0..Kp) = src[row][0..KR) followed by zeros
__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int KR, int Kp) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * Kp) return;
  const int row = i / Kp, k = i - row * Kp;
  dst[i] = k < KR ? src[(long long)row * KR + k] : 0.f;
}
// dst[row][0..KR) += src[row][0..KR)   (src rows are Kp long)
__global__ void fold_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int KR, int Kp) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * KR) return;
  const int row = i / KR, k = i - row * KR;
  dst[i] += src[(long long)row * Kp + k];
}

// the GEMM sees the patch matrix as a 1 x 1 x M "image" with Kp channels
XbConvGeom as_gemm(const XbConvGeom* g, int Kp, long long M) {
  XbConvGeom f{};
  f.N = 1; f.H = 1; f.W = (int)M; f.C = Kp; f.K = g->K; f.R = 1; f.S = 1; f.P = 1; f.Q = (int)M; f.sh = 1; f.sw = 1; f.ph = 0; f.pw = 0;
  return f;
}

int run_im2col(const float* X, float* A, const XbConvGeom* g, int Kp, long long M, cudaStream_t st) {
  if ((Kp >> 2) > 256) return -XB_BAD_ARG;
  const int per = 256 / (Kp >> 2);
  long long blocks = (M + (long long)per * 8 - 1) / ((long long)per * 8);      // ~8 positions per thread
  if (blocks > 148 * 16) blocks = 148 * 16;
  const int rows_per_block = (int)((M + blocks - 1) / blocks);
  blocks = (M + rows_per_block - 1) / rows_per_block;
  im2col_kernel<<<(unsigned)blocks, 256, 0, st>>>(X, A, *g, Kp, M, rows_per_block);
  return (int)cudaGetLastError();
}

}  // namespace

// which: 0 forward, 2 weight gradient.  Bytes of scratch the call needs, 0 if this path does not apply.
XB_API long long xb_conv_im2col_scratch(const XbConvGeom* g, int which) {
  if (which != 0 && which != 2) return 0;
  const long long M = (long long)g->N * g->P * g->Q;
  const int Kp = padded_k(g);
  if (M * Kp >= (1ll << 31) || M >= (1ll << 31) || g->K % 4 || Kp > 1024) return 0;
  XbConvGeom f = as_gemm(g, Kp, M);
  if (!xb_conv1x1_tma_supported(&f, which)) return 0;
  return (long long)(align256((size_t)M * Kp * 4) + align256((size_t)g->K * Kp * 4));
}

XB_API int xb_conv_fprop_im2col(const float* X, const float* W, const float* bias, float* Y, float* stats, const XbConvGeom* g, int flags,
                                float* scratch, int* status, cudaStream_t st) {
  if (!scratch || !xb_conv_im2col_scratch(g, 0)) return -XB_BAD_ARG;
  const long long M = (long long)g->N * g->P * g->Q;
  const int Kp = padded_k(g), KR = g->R * g->S * g->C;
  float* A = scratch;
  float* Wp = scratch + align256((size_t)M * Kp * 4) / 4;
  int e;
  if ((e = run_im2col(X, A, g, Kp, M, st))) return e;
  pad_rows_kernel<<<(g->K * Kp + 255) / 256, 256, 0, st>>>(W, Wp, g->K, KR, Kp);
  if ((e = (int)cudaGetLastError())) return e;
  XbConvGeom f = as_gemm(g, Kp, M);
  return xb_conv1x1_tma(A, Wp, bias, Y, stats, &f, 0, flags, status, st, nullptr);
}

// dW (K,R,S,C) += dY^T A; dW must hold the value to accumulate onto (normally zero).
// `reuse_patches` != 0: the scratch still holds this layer's patch matrix from the forward pass of the same task.
XB_API int xb_conv_wgrad_im2col(const float* dY, const float* X, float* dW, const XbConvGeom* g, float* scratch, int reuse_patches, int* status,
                                cudaStream_t st) {
  if (!scratch || !xb_conv_im2col_scratch(g, 2)) return -XB_BAD_ARG;
  const long long M = (long long)g->N * g->P * g->Q;
  const int Kp = padded_k(g), KR = g->R * g->S * g->C;
  float* A = scratch;
  float* dWp = scratch + align256((size_t)M * Kp * 4) / 4;
  int e;
  if (!reuse_patches && (e = run_im2col(X, A, g, Kp, M, st))) return e;
  if ((e = (int)cudaMemsetAsync(dWp, 0, (size_t)g->K * Kp * 4, st))) return e;
  XbConvGeom f = as_gemm(g, Kp, M);
  if ((e = xb_conv1x1_wgrad_tma(dY, A, dWp, &f, status, st))) return e;
  fold_rows_kernel<<<(g->K * KR + 255) / 256, 256, 0, st>>>(dWp, dW, g->K, KR, Kp);
  return (int)cudaGetLastError();
}
