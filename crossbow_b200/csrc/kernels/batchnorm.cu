// Spatial batch normalisation, channels-last, with ReLU and residual-add fused into the normalise pass.
//
// Training forward is two passes over x: (1) per-channel sum / sum of squares (often produced for free by the
// convolution epilogue, see igemm kernels), (2) normalise + scale/shift (+ residual) (+ ReLU).  Pass 2 also stores
// the batch mean / inverse std for the backward pass and blends the running statistics, which are ONE buffer per
// (operator, device) shared by all replicas on that device, as in the reference
// (clib-multigpu/kernels/cudnnbatchnorm.cu:99-151, cudnn/cudnnbatchnormparams.c:91-100).
// Backward is (1) per-channel sums of dz and dz*xhat, (2) dx (+ residual gradient) and dgamma/dbeta
// (cudnnbatchnormgradient.cu:77-93).  dz = dy masked by the fused ReLU.  The mask comes from one of three places: the
// layer's output y (> 0); x itself, re-normalised with the forward pass's own expressions (no residual input); or a
// packed sign mask the forward pass wrote next to y - one byte per four channels, a sixteenth of y's size - which is what
// layers with a residual input use, so that neither backward pass reads y.
//
// Thread mapping: a thread keeps the same 4 channels for its whole life ("column-persistent"), so the per-channel
// constants are computed once and rows are streamed with 16-byte loads.
#include "common.cuh"

namespace {

constexpr int NT = 256;

template <int VEC> struct VecT;
template <> struct VecT<4> { using T = float4; };
template <> struct VecT<1> { using T = float; };

template <int VEC> __device__ __forceinline__ void ld(const float* p, float (&v)[VEC]) {
  if constexpr (VEC == 4) { float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  else v[0] = *p;
}
template <int VEC> __device__ __forceinline__ void st(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}

// Column-persistent iteration space: CV = C/VEC column groups; a block covers `rows_per_iter` rows per step.
struct Tiling { int cv, rows_per_iter, col_passes; };
__host__ __device__ inline Tiling make_tiling(int C, int vec) {
  Tiling t; t.cv = C / vec;
  if (t.cv >= NT) { t.rows_per_iter = 1; t.col_passes = (t.cv + NT - 1) / NT; }
  else { t.rows_per_iter = NT / t.cv; t.col_passes = 1; }
  return t;
}

// sums[0..C) += sum_x, sums[C..2C) += sum_x^2 ; optionally of a*(mask) for backward
template <int VEC>
__global__ void __launch_bounds__(NT) bn_stats_kernel(const float* __restrict__ x, float* __restrict__ sums, int M, int C, int rows_per_block) {
  xb_pdl_wait();
  xb_pdl_launch();
  const Tiling t = make_tiling(C, VEC);
  __shared__ float red[2][NT * VEC];
  const int r_begin = blockIdx.x * rows_per_block, r_end = min(M, r_begin + rows_per_block);
  for (int pass = 0; pass < t.col_passes; ++pass) {
    int cg = (t.col_passes == 1) ? (threadIdx.x % t.cv) : (pass * NT + threadIdx.x);
    int rsub = (t.col_passes == 1) ? (threadIdx.x / t.cv) : 0;
    bool active = cg < t.cv && rsub < t.rows_per_iter;
    float s[VEC], q[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) { s[e] = 0.f; q[e] = 0.f; }
    if (active)
      for (int r = r_begin + rsub; r < r_end; r += t.rows_per_iter) {
        float v[VEC]; ld<VEC>(x + (long long)r * C + cg * VEC, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) { s[e] += v[e]; q[e] += v[e] * v[e]; }
      }
    // reduce over rsub within the block
#pragma unroll
    for (int e = 0; e < VEC; ++e) { red[0][threadIdx.x * VEC + e] = s[e]; red[1][threadIdx.x * VEC + e] = q[e]; }
    __syncthreads();
    if (active && rsub == 0) {
      for (int j = 1; j < t.rows_per_iter; ++j) {
        int o = (threadIdx.x + j * t.cv) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) { s[e] += red[0][o + e]; q[e] += red[1][o + e]; }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) { atomicAdd(&sums[cg * VEC + e], s[e]); atomicAdd(&sums[C + cg * VEC + e], q[e]); }
    }
    __syncthreads();
  }
}

struct BnArgs {
  const float* x; const float* res; float* y;
  const float* sums;              // training: sum, sumsq [2C]
  const float* gamma; const float* beta;
  float* run_mean; float* run_var;
  float* save_mean; float* save_invstd;
  const XbTaskParams* tp;
  int M, C; float eps; int relu; int training; int cma; float fraction_factor;
  int rows_per_block;
  unsigned char* mask;            // VEC == 4 only, may be null: bit e of byte (row * C + c) / 4 = (y[c + e] > 0)
};

template <int VEC>
__global__ void __launch_bounds__(NT) bn_fwd_kernel(BnArgs a) {
  xb_pdl_wait();
  xb_pdl_launch();
  const Tiling t = make_tiling(a.C, VEC);
  const int r_begin = blockIdx.x * a.rows_per_block, r_end = min(a.M, r_begin + a.rows_per_block);
  const float invM = 1.f / (float)a.M;
  for (int pass = 0; pass < t.col_passes; ++pass) {
    int cg = (t.col_passes == 1) ? (threadIdx.x % t.cv) : (pass * NT + threadIdx.x);
    int rsub = (t.col_passes == 1) ? (threadIdx.x / t.cv) : 0;
    if (cg >= t.cv || rsub >= t.rows_per_iter) continue;
    float sc[VEC], sh[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      int c = cg * VEC + e;
      float mean, invstd;
      if (a.training) {
        mean = a.sums[c] * invM;
        float var = fmaxf(a.sums[a.C + c] * invM - mean * mean, 0.f);
        invstd = rsqrtf(var + a.eps);
        if (blockIdx.x == 0 && rsub == 0) {
          a.save_mean[c] = mean; a.save_invstd[c] = invstd;
          float f = a.cma ? a.tp->bn_factor : a.fraction_factor;
          float unb = var * ((float)a.M / (float)max(1, a.M - 1));
          // shared by all replicas of the device: blend with atomics so concurrent learners do not tear values
          atomicAdd(&a.run_mean[c], f * (mean - a.run_mean[c]));
          atomicAdd(&a.run_var[c], f * (unb - a.run_var[c]));
        }
      } else {
        mean = a.run_mean[c];
        invstd = rsqrtf(a.run_var[c] + a.eps);
      }
      // explicit fused multiply-adds: the backward pass re-derives the ReLU mask from x with the same two expressions
      sc[e] = a.gamma[c] * invstd;
      sh[e] = __fmaf_rn(-mean, sc[e], a.beta[c]);
    }
    constexpr int RU = 4;                                // rows per step: all loads first, then the stores
    const long long step = (long long)t.rows_per_iter * a.C;
    int r = r_begin + rsub;
    for (; r + (RU - 1) * t.rows_per_iter < r_end; r += RU * t.rows_per_iter) {
      const long long off = (long long)r * a.C + cg * VEC;
      float v[RU][VEC], rr[RU][VEC];
#pragma unroll
      for (int u = 0; u < RU; ++u) ld<VEC>(a.x + off + u * step, v[u]);
      if (a.res) {
#pragma unroll
        for (int u = 0; u < RU; ++u) ld<VEC>(a.res + off + u * step, rr[u]);
      }
#pragma unroll
      for (int u = 0; u < RU; ++u) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float o = __fmaf_rn(v[u][e], sc[e], sh[e]);
          if (a.res) o += rr[u][e];
          if (a.relu) o = fmaxf(o, 0.f);
          v[u][e] = o;
        }
        st<VEC>(a.y + off + u * step, v[u]);
        if constexpr (VEC == 4) {
          if (a.mask) a.mask[(off + u * step) >> 2] = (unsigned char)((v[u][0] > 0.f) | ((v[u][1] > 0.f) << 1) | ((v[u][2] > 0.f) << 2) | ((v[u][3] > 0.f) << 3));
        }
      }
    }
    for (; r < r_end; r += t.rows_per_iter) {
      long long off = (long long)r * a.C + cg * VEC;
      float v[VEC]; ld<VEC>(a.x + off, v);
      float rr[VEC];
      if (a.res) ld<VEC>(a.res + off, rr);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float o = __fmaf_rn(v[e], sc[e], sh[e]);
        if (a.res) o += rr[e];
        if (a.relu) o = fmaxf(o, 0.f);
        v[e] = o;
      }
      st<VEC>(a.y + off, v);
      if constexpr (VEC == 4) {
        if (a.mask) a.mask[off >> 2] = (unsigned char)((v[0] > 0.f) | ((v[1] > 0.f) << 1) | ((v[2] > 0.f) << 2) | ((v[3] > 0.f) << 3));
      }
    }
  }
}

struct BnBwdArgs {
  const float* dy; const float* x; const float* y;   // y = forward output (ReLU mask) or null
  const float* save_mean; const float* save_invstd; const float* gamma;
  float* dsums;                                      // [2C]: sum dz, sum dz*xhat
  float* dx; float* dres; float* dgamma; float* dbeta;
  int M, C; int relu; int accum_dx; int accum_dres; int rows_per_block;   // relu == 3: `y` is the packed sign mask (bytes)
  const float* beta;   // relu == 2: the mask is re-derived from x (fma(x, gamma*istd, beta - mean*gamma*istd) > 0) and y is not read
};

// MODE: where the ReLU mask comes from - 0 none, 1 the output y, 2 re-derived from x, 3 the packed sign bytes; -1 = read
// it from the arguments at run time (the scalar kernels).  A compile-time mode keeps the registers of the unused mask
// sources out of the kernel, which is what lets three blocks share an SM.
template <int VEC, int MODE = -1>
__global__ void __launch_bounds__(NT, MODE >= 0 ? 3 : 1) bn_bwd_reduce_kernel(BnBwdArgs a) {
  xb_pdl_wait();
  xb_pdl_launch();
  const Tiling t = make_tiling(a.C, VEC);
  __shared__ float red[2][NT * VEC];
  const int r_begin = blockIdx.x * a.rows_per_block, r_end = min(a.M, r_begin + a.rows_per_block);
  for (int pass = 0; pass < t.col_passes; ++pass) {
    int cg = (t.col_passes == 1) ? (threadIdx.x % t.cv) : (pass * NT + threadIdx.x);
    int rsub = (t.col_passes == 1) ? (threadIdx.x / t.cv) : 0;
    bool active = cg < t.cv && rsub < t.rows_per_iter;
    float s1[VEC], s2[VEC], mean[VEC], istd[VEC], msc[VEC], msh[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) { s1[e] = 0.f; s2[e] = 0.f; mean[e] = 0.f; istd[e] = 0.f; msc[e] = 0.f; msh[e] = 0.f; }
    const int mode = MODE >= 0 ? MODE : a.relu;
    const bool from_y = mode == 1, from_x = mode == 2, from_m = (VEC == 4) && mode == 3;
    const unsigned char* mk = reinterpret_cast<const unsigned char*>(a.y);
    if (active) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        mean[e] = a.save_mean[cg * VEC + e]; istd[e] = a.save_invstd[cg * VEC + e];
        if (from_x) { msc[e] = a.gamma[cg * VEC + e] * istd[e]; msh[e] = __fmaf_rn(-mean[e], msc[e], a.beta[cg * VEC + e]); }
      }
      // four rows per step: twelve 16-byte loads in flight per thread before the first use
      constexpr int RU = 4;
      const long long step = (long long)t.rows_per_iter * a.C;
      int r = r_begin + rsub;
      for (; r + (RU - 1) * t.rows_per_iter < r_end; r += RU * t.rows_per_iter) {
        const long long off = (long long)r * a.C + cg * VEC;
        float g[RU][VEC], xv[RU][VEC], yv[RU][VEC];
        unsigned int mb[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) { ld<VEC>(a.dy + off + u * step, g[u]); ld<VEC>(a.x + off + u * step, xv[u]); mb[u] = 0; }
        if (from_y) {
#pragma unroll
          for (int u = 0; u < RU; ++u) ld<VEC>(a.y + off + u * step, yv[u]);
        }
        if (from_m) {
#pragma unroll
          for (int u = 0; u < RU; ++u) mb[u] = mk[(off + u * step) >> 2];
        }
#pragma unroll
        for (int u = 0; u < RU; ++u)
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            const bool off_ = from_m ? !((mb[u] >> e) & 1u) : from_y ? !(yv[u][e] > 0.f) : (from_x && !(__fmaf_rn(xv[u][e], msc[e], msh[e]) > 0.f));
            float dz = off_ ? 0.f : g[u][e];
            s1[e] += dz; s2[e] += dz * (xv[u][e] - mean[e]) * istd[e];
          }
      }
      for (; r < r_end; r += t.rows_per_iter) {
        long long off = (long long)r * a.C + cg * VEC;
        float g[VEC], xv[VEC], yv[VEC];
        ld<VEC>(a.dy + off, g); ld<VEC>(a.x + off, xv);
        if (from_y) ld<VEC>(a.y + off, yv);
        const unsigned int mb = from_m ? mk[off >> 2] : 0u;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const bool off_ = from_m ? !((mb >> e) & 1u) : from_y ? !(yv[e] > 0.f) : (from_x && !(__fmaf_rn(xv[e], msc[e], msh[e]) > 0.f));
          float dz = off_ ? 0.f : g[e];
          s1[e] += dz; s2[e] += dz * (xv[e] - mean[e]) * istd[e];
        }
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) { red[0][threadIdx.x * VEC + e] = s1[e]; red[1][threadIdx.x * VEC + e] = s2[e]; }
    __syncthreads();
    if (active && rsub == 0) {
      for (int j = 1; j < t.rows_per_iter; ++j) {
        int o = (threadIdx.x + j * t.cv) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) { s1[e] += red[0][o + e]; s2[e] += red[1][o + e]; }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) { atomicAdd(&a.dsums[cg * VEC + e], s1[e]); atomicAdd(&a.dsums[a.C + cg * VEC + e], s2[e]); }
    }
    __syncthreads();
  }
}

template <int VEC>
__global__ void __launch_bounds__(NT) bn_bwd_apply_kernel(BnBwdArgs a) {
  xb_pdl_wait();
  xb_pdl_launch();
  const Tiling t = make_tiling(a.C, VEC);
  const int r_begin = blockIdx.x * a.rows_per_block, r_end = min(a.M, r_begin + a.rows_per_block);
  const float invM = 1.f / (float)a.M;
  for (int pass = 0; pass < t.col_passes; ++pass) {
    int cg = (t.col_passes == 1) ? (threadIdx.x % t.cv) : (pass * NT + threadIdx.x);
    int rsub = (t.col_passes == 1) ? (threadIdx.x / t.cv) : 0;
    if (cg >= t.cv || rsub >= t.rows_per_iter) continue;
    float mean[VEC], istd[VEC], k0[VEC], k1[VEC], k2[VEC], msh[VEC];
    const bool from_y = a.relu == 1, from_x = a.relu == 2, from_m = (VEC == 4) && a.relu == 3;
    const unsigned char* mk = reinterpret_cast<const unsigned char*>(a.y);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      int c = cg * VEC + e;
      mean[e] = a.save_mean[c]; istd[e] = a.save_invstd[c];
      float s1 = a.dsums[c], s2 = a.dsums[a.C + c];
      float gi = a.gamma[c] * istd[e];
      msh[e] = from_x ? __fmaf_rn(-mean[e], gi, a.beta[c]) : 0.f;       // (gi = gamma * istd is the forward pass's scale)
      k0[e] = gi; k1[e] = gi * s1 * invM; k2[e] = gi * s2 * invM;
      if (blockIdx.x == 0 && rsub == 0) { atomicAdd(&a.dgamma[c], s2); atomicAdd(&a.dbeta[c], s1); }
    }
    for (int r = r_begin + rsub; r < r_end; r += t.rows_per_iter) {
      long long off = (long long)r * a.C + cg * VEC;
      float g[VEC], xv[VEC], yv[VEC], o[VEC], old[VEC];
      ld<VEC>(a.dy + off, g); ld<VEC>(a.x + off, xv);
      if (from_y) ld<VEC>(a.y + off, yv);
      const unsigned int mb = from_m ? mk[off >> 2] : 0u;
      if (a.accum_dx) ld<VEC>(a.dx + off, old);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const bool off_ = from_m ? !((mb >> e) & 1u) : from_y ? !(yv[e] > 0.f) : (from_x && !(__fmaf_rn(xv[e], k0[e], msh[e]) > 0.f));
        float dz = off_ ? 0.f : g[e];
        g[e] = dz;
        float xhat = (xv[e] - mean[e]) * istd[e];
        o[e] = k0[e] * dz - k1[e] - k2[e] * xhat;
        if (a.accum_dx) o[e] += old[e];
      }
      st<VEC>(a.dx + off, o);
      if (a.dres) {
        if (a.accum_dres) {
          float rr[VEC]; ld<VEC>(a.dres + off, rr);
#pragma unroll
          for (int e = 0; e < VEC; ++e) g[e] += rr[e];
        }
        st<VEC>(a.dres + off, g);
      }
    }
  }
}

template <class A> static void launch_reduce_v4(const A& a, int blocks, cudaStream_t st) {
  switch (a.relu) {
    case 0: xb_launch(bn_bwd_reduce_kernel<4, 0>, dim3(blocks), dim3(NT), 0, st, a); break;
    case 1: xb_launch(bn_bwd_reduce_kernel<4, 1>, dim3(blocks), dim3(NT), 0, st, a); break;
    case 2: xb_launch(bn_bwd_reduce_kernel<4, 2>, dim3(blocks), dim3(NT), 0, st, a); break;
    default: xb_launch(bn_bwd_reduce_kernel<4, 3>, dim3(blocks), dim3(NT), 0, st, a); break;
  }
}

// Reductions end in 2C same-address atomics per block, which serialise in L2: they get fewer, longer blocks.
static int g_bn_reduce_blocks = 296;
static int g_bn_stream_blocks = 592;                   // normalise / apply passes (no atomics): ~4 resident blocks per SM
inline int rows_per_block_for(int M, int C, int vec, int& blocks, int target = 0, int min_steps = 2) {
  // small tensors (<= 8 MB) are latency-bound and run better with half as many, longer blocks
  if (target <= 0) target = ((long long)M * C <= (2ll << 20)) ? g_bn_stream_blocks / 2 : g_bn_stream_blocks;
  Tiling t = make_tiling(C, vec);
  // aim for ~4 resident blocks per SM (592 blocks), at least 2 row-steps per block
  int min_rows = t.rows_per_iter * min_steps;
  int rpb = xb_ceil_div(M, target);
  if (rpb < min_rows) rpb = min_rows;
  rpb = xb_ceil_div(rpb, t.rows_per_iter) * t.rows_per_iter;
  blocks = xb_ceil_div(M, rpb);
  return rpb;
}

inline bool can_vec4(int C, const void* a, const void* b, const void* c, const void* d) {
  return (C % 4 == 0) && ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)d)) % 16 == 0);
}

}  // namespace

XB_API int xb_bn_stats(const float* x, float* sums, int M, int C, cudaStream_t st) {
  bool v4 = can_vec4(C, x, nullptr, nullptr, nullptr);
  int blocks; int rpb = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) xb_launch(bn_stats_kernel<4>, dim3(blocks), dim3(NT), 0, st, x, sums, M, C, rpb);
  else    xb_launch(bn_stats_kernel<1>, dim3(blocks), dim3(NT), 0, st, x, sums, M, C, rpb);
  return (int)cudaGetLastError();
}

// `mask` (may be null; needs C % 4 == 0 and 16-byte aligned tensors): M * C / 4 bytes that receive the signs of y, four
// channels per byte, for xb_bn_backward with relu == 3.
XB_API int xb_bn_forward_mask(const float* x, const float* res, float* y, const float* sums, const float* gamma, const float* beta,
                              float* run_mean, float* run_var, float* save_mean, float* save_invstd, const XbTaskParams* tp,
                              int M, int C, float eps, int relu, int training, int cma, float fraction_factor, unsigned char* mask,
                              cudaStream_t st);
XB_API int xb_bn_forward(const float* x, const float* res, float* y, const float* sums, const float* gamma, const float* beta,
                         float* run_mean, float* run_var, float* save_mean, float* save_invstd, const XbTaskParams* tp,
                         int M, int C, float eps, int relu, int training, int cma, float fraction_factor, cudaStream_t st) {
  return xb_bn_forward_mask(x, res, y, sums, gamma, beta, run_mean, run_var, save_mean, save_invstd, tp, M, C, eps, relu, training, cma,
                            fraction_factor, nullptr, st);
}
XB_API int xb_bn_forward_mask(const float* x, const float* res, float* y, const float* sums, const float* gamma, const float* beta,
                              float* run_mean, float* run_var, float* save_mean, float* save_invstd, const XbTaskParams* tp,
                              int M, int C, float eps, int relu, int training, int cma, float fraction_factor, unsigned char* mask,
                              cudaStream_t st) {
  BnArgs a{x, res, y, sums, gamma, beta, run_mean, run_var, save_mean, save_invstd, tp, M, C, eps, relu, training, cma, fraction_factor, 0, mask};
  bool v4 = can_vec4(C, x, res, y, nullptr);
  if (mask && !v4) return -XB_BAD_ARG;
  int blocks; a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) xb_launch(bn_fwd_kernel<4>, dim3(blocks), dim3(NT), 0, st, a);
  else    xb_launch(bn_fwd_kernel<1>, dim3(blocks), dim3(NT), 0, st, a);
  return (int)cudaGetLastError();
}

// dsums must be zero on entry.  dgamma/dbeta are accumulated (+=).
XB_API int xb_bn_backward(const float* dy, const float* x, const float* y, const float* save_mean, const float* save_invstd,
                          const float* gamma, float* dsums, float* dx, float* dres, float* dgamma, float* dbeta,
                          int M, int C, int relu, int accum_dx, int accum_dres, cudaStream_t st) {
  // relu: 0 none, 1 mask from y (> 0), 3 `y` is the packed sign mask written by xb_bn_forward_mask
  BnBwdArgs a{dy, x, y, save_mean, save_invstd, gamma, dsums, dx, dres, dgamma, dbeta, M, C, relu == 3 ? 3 : (relu ? 1 : 0), accum_dx, accum_dres, 0, nullptr};
  bool v4 = can_vec4(C, dy, x, relu == 3 ? nullptr : y, dx) && (((uintptr_t)dres) % 16 == 0);
  if (relu == 3 && !v4) return -XB_BAD_ARG;
  int blocks, rblocks; a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, rblocks, g_bn_reduce_blocks, 8);
  if (v4) launch_reduce_v4(a, rblocks, st); else xb_launch(bn_bwd_reduce_kernel<1>, dim3(rblocks), dim3(NT), 0, st, a);
  a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) xb_launch(bn_bwd_apply_kernel<4>, dim3(blocks), dim3(NT), 0, st, a); else xb_launch(bn_bwd_apply_kernel<1>, dim3(blocks), dim3(NT), 0, st, a);
  return (int)cudaGetLastError();
}
XB_API void xb_bn_set_reduce_blocks(int n) { g_bn_reduce_blocks = n > 0 ? n : 296; }
XB_API void xb_bn_set_stream_blocks(int n) { g_bn_stream_blocks = n > 0 ? n : 592; }

// As xb_bn_backward, for a layer whose fused ReLU has no residual input: the mask is re-derived from x, gamma, beta and the
// saved statistics with the forward pass's own expressions (bit-identical), so the layer's output is not read at all -
// five passes over the tensor instead of seven.
XB_API int xb_bn_backward_remask(const float* dy, const float* x, const float* save_mean, const float* save_invstd, const float* gamma,
                                 const float* beta, float* dsums, float* dx, float* dgamma, float* dbeta, int M, int C, int accum_dx,
                                 cudaStream_t st) {
  BnBwdArgs a{dy, x, nullptr, save_mean, save_invstd, gamma, dsums, dx, nullptr, dgamma, dbeta, M, C, 2, accum_dx, 0, 0, beta};
  bool v4 = can_vec4(C, dy, x, nullptr, dx);
  int blocks, rblocks; a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, rblocks, g_bn_reduce_blocks, 8);
  if (v4) launch_reduce_v4(a, rblocks, st); else xb_launch(bn_bwd_reduce_kernel<1>, dim3(rblocks), dim3(NT), 0, st, a);
  a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) xb_launch(bn_bwd_apply_kernel<4>, dim3(blocks), dim3(NT), 0, st, a); else xb_launch(bn_bwd_apply_kernel<1>, dim3(blocks), dim3(NT), 0, st, a);
  return (int)cudaGetLastError();
}

// Second half only: `dsums` already holds the sums (produced by the epilogue of the kernel that completed dy).
XB_API int xb_bn_backward_apply(const float* dy, const float* x, const float* y, const float* save_mean, const float* save_invstd,
                                const float* gamma, const float* dsums, float* dx, float* dres, float* dgamma, float* dbeta,
                                int M, int C, int relu, int accum_dx, int accum_dres, cudaStream_t st) {
  BnBwdArgs a{dy, x, y, save_mean, save_invstd, gamma, const_cast<float*>(dsums), dx, dres, dgamma, dbeta, M, C, relu ? 1 : 0, accum_dx, accum_dres, 0, nullptr};
  bool v4 = can_vec4(C, dy, x, y, dx) && (((uintptr_t)dres) % 16 == 0);
  int blocks; a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) xb_launch(bn_bwd_apply_kernel<4>, dim3(blocks), dim3(NT), 0, st, a);
  else    xb_launch(bn_bwd_apply_kernel<1>, dim3(blocks), dim3(NT), 0, st, a);
  return (int)cudaGetLastError();
}

// ---- variant that allocates nothing: the scratch sums live in a fixed device array (see bn_backward_static.h) ----------
#include "bn_backward_static.h"
#include <stdio.h>

// 2 * XB_BN_STATIC_MAX_CHANNELS floats = 32 KB per GPU, resident for the life of the process.  In host code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_bn_static_sums[2 * XB_BN_STATIC_MAX_CHANNELS];

#include <atomic>
namespace {
constexpr int kMaxDevices = 64;
// device address of the array, per device, filled on first use; atomic because several host threads may make their
// first call on a device at the same time (they all store the same value)
std::atomic<float*> g_bn_static_ptr[kMaxDevices];
}

extern "C" __attribute__((visibility("default")))
int xb_bn_backward_static(const float* dy, const float* x, const float* y, const float* save_mean, const float* save_invstd,
                          const float* gamma, float* dx, float* dres, float* dgamma, float* dbeta, int M, int C, int relu,
                          int accum_dx, int accum_dres, cudaStream_t stream) {
  if (C > XB_BN_STATIC_MAX_CHANNELS) {
    fprintf(stderr, "xb_bn_backward_static: %d channels exceed the built-in scratch of %d channels; use xb_bn_backward with your own scratch\n",
            C, XB_BN_STATIC_MAX_CHANNELS);
    return XB_BN_STATIC_TOO_MANY_CHANNELS;
  }
  if (M <= 0 || C <= 0 || !dy || !x || !dx || !dgamma || !dbeta || !save_mean || !save_invstd || !gamma || (relu && !y))
    return XB_BN_STATIC_BAD_ARGUMENT;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return XB_BN_STATIC_BAD_ARGUMENT;
  float* sums = g_bn_static_ptr[dev].load(std::memory_order_acquire);
  if (!sums) {
    // once per device, with that device current: translate the symbol into the address the kernels can use
    e = cudaGetSymbolAddress((void**)&sums, g_bn_static_sums);
    if (e != cudaSuccess) return (int)e;
    g_bn_static_ptr[dev].store(sums, std::memory_order_release);
  }
  e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * (size_t)C, stream);     // the sums accumulate from zero
  if (e != cudaSuccess) return (int)e;
  BnBwdArgs a{dy, x, y, save_mean, save_invstd, gamma, sums, dx, dres, dgamma, dbeta, M, C, relu ? 1 : 0, accum_dx, accum_dres, 0, nullptr};
  bool v4 = can_vec4(C, dy, x, y, dx) && (((uintptr_t)dres) % 16 == 0);
  // same launch shapes as xb_bn_backward: fewer, longer blocks for the reduction (its tail is same-address atomics)
  int blocks, rblocks; a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, rblocks, g_bn_reduce_blocks, 8);
  if (v4) launch_reduce_v4(a, rblocks, stream); else bn_bwd_reduce_kernel<1><<<rblocks, NT, 0, stream>>>(a);
  a.rows_per_block = rows_per_block_for(M, C, v4 ? 4 : 1, blocks);
  if (v4) bn_bwd_apply_kernel<4><<<blocks, NT, 0, stream>>>(a); else bn_bwd_apply_kernel<1><<<blocks, NT, 0, stream>>>(a);
  return (int)cudaGetLastError();
}
