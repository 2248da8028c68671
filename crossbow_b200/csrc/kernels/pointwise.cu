// Element-wise operators, channels-last: activations, weighted sums, dropout, channel concat / slice, pooling,
// local response normalisation, input transform.  Each replaces a cuDNN / cuBLAS call of the reference:
//   cudnnrelu.cu / cudnnrelugradient.cu, elementwiseop.cu / elementwiseopgradient.cu (saxpy per input),
//   cudnndropout.cu / cudnndropoutgradient.cu, concat.cu / concatgradient.cu, cudnnpool.cu / cudnnpoolgradient.cu,
//   datatransform.cu.  LRN has no GPU implementation in the reference (executioncontext.c:374,395).
#include "common.cuh"
#include <float.h>
#include <string.h>

namespace {
constexpr int NT = 256;
inline int grid_for(long long n, int per_thread = 1) {
  long long b = (n + (long long)NT * per_thread - 1) / ((long long)NT * per_thread);
  if (b > 148 * 32) b = 148 * 32;
  if (b < 1) b = 1;
  return (int)b;
}

// mode: 0 sigmoid, 1 relu (with negative slope), 2 tanh, 3 clipped relu
__global__ void act_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, int mode, float slope, float ceiling) {
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    float v = x[i], o;
    if (mode == 1) o = v > 0.f ? v : v * slope;
    else if (mode == 0) o = 1.f / (1.f + __expf(-v));
    else if (mode == 2) o = tanhf(v);
    else o = fminf(fmaxf(v, 0.f), ceiling);
    y[i] = o;
  }
}
__global__ void act_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ y,
                               float* __restrict__ dx, long long n, int mode, float slope, float ceiling, int accum) {
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    float g = dy[i], o;
    if (mode == 1) o = y[i] > 0.f ? g : g * slope;      // y>0 <=> x>0 for slope>=0
    else if (mode == 0) { float s = y[i]; o = g * s * (1.f - s); }
    else if (mode == 2) { float t = y[i]; o = g * (1.f - t * t); }
    else { float v = x[i]; o = (v > 0.f && v < ceiling) ? g : 0.f; }
    dx[i] = accum ? dx[i] + o : o;
  }
}

__device__ __forceinline__ float act_one(float v, int mode, float slope, float ceiling) {
  if (mode == 1) return v > 0.f ? v : v * slope;
  if (mode == 0) return 1.f / (1.f + __expf(-v));
  if (mode == 2) return tanhf(v);
  return fminf(fmaxf(v, 0.f), ceiling);
}
__device__ __forceinline__ float act_grad_one(float g, float x, float y, int mode, float slope, float ceiling) {
  if (mode == 1) return y > 0.f ? g : g * slope;
  if (mode == 0) return g * y * (1.f - y);
  if (mode == 2) return g * (1.f - y * y);
  return (x > 0.f && x < ceiling) ? g : 0.f;
}
// 16-byte forms of the two kernels above (n4 = elements / 4, all pointers 16-byte aligned)
__global__ void act_fwd_v4_kernel(const float4* __restrict__ x, float4* __restrict__ y, long long n4, int mode, float slope, float ceiling) {
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n4; i += (long long)gridDim.x * NT) {
    const float4 v = x[i];
    y[i] = make_float4(act_one(v.x, mode, slope, ceiling), act_one(v.y, mode, slope, ceiling), act_one(v.z, mode, slope, ceiling),
                       act_one(v.w, mode, slope, ceiling));
  }
}
__global__ void act_bwd_v4_kernel(const float4* __restrict__ dy, const float4* __restrict__ x, const float4* __restrict__ y,
                                  float4* __restrict__ dx, long long n4, int mode, float slope, float ceiling, int accum) {
  const bool need_x = mode == 3;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n4; i += (long long)gridDim.x * NT) {
    const float4 g = dy[i], yy = y[i];
    const float4 xx = need_x ? x[i] : yy;
    float4 o = make_float4(act_grad_one(g.x, xx.x, yy.x, mode, slope, ceiling), act_grad_one(g.y, xx.y, yy.y, mode, slope, ceiling),
                           act_grad_one(g.z, xx.z, yy.z, mode, slope, ceiling), act_grad_one(g.w, xx.w, yy.w, mode, slope, ceiling));
    if (accum) { const float4 d = dx[i]; o.x += d.x; o.y += d.y; o.z += d.z; o.w += d.w; }
    dx[i] = o;
  }
}

// y = (accum ? y : 0) + sum_i coef[i]*x[i]
struct SumArgs { const float* x[4]; float coef[4]; int n_in; };
__global__ void weighted_sum_kernel(SumArgs a, float* __restrict__ y, long long n4, long long n, int accum) {
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n4; i += (long long)gridDim.x * NT) {
    float4 o = accum ? reinterpret_cast<float4*>(y)[i] : make_float4(0, 0, 0, 0);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < a.n_in) {
        float4 v = reinterpret_cast<const float4*>(a.x[k])[i];
        o.x = fmaf(a.coef[k], v.x, o.x); o.y = fmaf(a.coef[k], v.y, o.y); o.z = fmaf(a.coef[k], v.z, o.z); o.w = fmaf(a.coef[k], v.w, o.w);
      }
    reinterpret_cast<float4*>(y)[i] = o;
  }
  // tail
  for (long long t = n4 * 4 + blockIdx.x * (long long)NT + threadIdx.x; t < n; t += (long long)gridDim.x * NT) {
    float o = accum ? y[t] : 0.f;
    for (int k = 0; k < a.n_in; ++k) o = fmaf(a.coef[k], a.x[k][t], o);
    y[t] = o;
  }
}

// Inverted dropout. Element i uses lane i%4 of Philox(counter = i/4, task, stream); keep iff u >= ratio.
__global__ void dropout_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, float ratio, unsigned stream,
                               const XbTaskParams* __restrict__ tp, int accum, bool vec) {
  const float scale = 1.f / (1.f - ratio);
  const unsigned task = tp->task_id, k0 = tp->seed_lo, k1 = tp->seed_hi;
  long long groups = (n + 3) / 4;
  for (long long gidx = blockIdx.x * (long long)NT + threadIdx.x; gidx < groups; gidx += (long long)gridDim.x * NT) {
    uint4 r = xb_philox4x32((uint32_t)gidx, task, stream, 0u, k0, k1);
    uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    if (vec && gidx * 4 + 3 < n) {          // one 16-byte load and store per group
      const float4 v = reinterpret_cast<const float4*>(x)[gidx];
      float4 o = make_float4((xb_u24(rr[0]) >= ratio) ? v.x * scale : 0.f, (xb_u24(rr[1]) >= ratio) ? v.y * scale : 0.f,
                             (xb_u24(rr[2]) >= ratio) ? v.z * scale : 0.f, (xb_u24(rr[3]) >= ratio) ? v.w * scale : 0.f);
      if (accum) { const float4 d = reinterpret_cast<const float4*>(y)[gidx]; o.x += d.x; o.y += d.y; o.z += d.z; o.w += d.w; }
      reinterpret_cast<float4*>(y)[gidx] = o;
      continue;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      long long i = gidx * 4 + e;
      if (i < n) {
        float o = (xb_u24(rr[e]) >= ratio) ? x[i] * scale : 0.f;
        y[i] = accum ? y[i] + o : o;
      }
    }
  }
}

// copy a [M, Cs] matrix into / out of columns [coff, coff+Cs) of a [M, Ct] matrix
__global__ void concat_copy_kernel(const float* __restrict__ src, float* __restrict__ dst, long long M, int Cs, int Ct, int coff, int to_wide, int accum) {
  long long n = M * Cs;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    long long m = i / Cs; int c = (int)(i % Cs);
    long long wide = m * Ct + coff + c;
    if (to_wide) dst[wide] = src[i];
    else dst[i] = accum ? dst[i] + src[wide] : src[wide];
  }
}

struct PoolGeom { int N, H, W, C, P, Q, kh, kw, sh, sw, ph, pw; };

// max pooling forward: first maximum wins (NaN propagates as in cuDNN's PROPAGATE_NAN only if it is the first element)
__global__ void maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, PoolGeom g) {
  long long n = (long long)g.N * g.P * g.Q * g.C;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int c = (int)(i % g.C); long long t = i / g.C; int q = (int)(t % g.Q); t /= g.Q; int p = (int)(t % g.P); int b = (int)(t / g.P);
    float best = -FLT_MAX;
    for (int r = 0; r < g.kh; ++r) {
      int iy = p * g.sh - g.ph + r; if (iy < 0 || iy >= g.H) continue;
      for (int s = 0; s < g.kw; ++s) {
        int ix = q * g.sw - g.pw + s; if (ix < 0 || ix >= g.W) continue;
        float v = x[(((long long)b * g.H + iy) * g.W + ix) * g.C + c];
        if (v > best) best = v;
      }
    }
    y[i] = best;
  }
}
// dx must be zeroed (or hold values to accumulate onto)
__global__ void maxpool_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, float* __restrict__ dx, PoolGeom g) {
  long long n = (long long)g.N * g.P * g.Q * g.C;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int c = (int)(i % g.C); long long t = i / g.C; int q = (int)(t % g.Q); t /= g.Q; int p = (int)(t % g.P); int b = (int)(t / g.P);
    float best = -FLT_MAX; long long arg = -1;
    for (int r = 0; r < g.kh; ++r) {
      int iy = p * g.sh - g.ph + r; if (iy < 0 || iy >= g.H) continue;
      for (int s = 0; s < g.kw; ++s) {
        int ix = q * g.sw - g.pw + s; if (ix < 0 || ix >= g.W) continue;
        long long o = (((long long)b * g.H + iy) * g.W + ix) * g.C + c;
        float v = x[o];
        if (v > best) { best = v; arg = o; }
      }
    }
    if (arg >= 0) atomicAdd(&dx[arg], dy[i]);
  }
}
// ---- 16-byte forms (C % 4 == 0, fewer than 2^31 groups): one thread = four channels of one output position -----------
template <bool AVG>
__global__ void __launch_bounds__(NT) pool_fwd_v4_kernel(const float4* __restrict__ x, float4* __restrict__ y, PoolGeom g) {
  const unsigned C4 = (unsigned)g.C >> 2, n = (unsigned)g.N * g.P * g.Q * C4;
  const float inv = 1.f / (float)(g.kh * g.kw);
  for (unsigned i = blockIdx.x * NT + threadIdx.x; i < n; i += gridDim.x * NT) {
    const unsigned c = i % C4; unsigned t = i / C4; const int q = t % g.Q; t /= g.Q; const int p = t % g.P, b = t / g.P;
    const int y0 = p * g.sh - g.ph, x0 = q * g.sw - g.pw;
    float4 a = AVG ? make_float4(0, 0, 0, 0) : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
    for (int r = 0; r < g.kh; ++r) {
      const int iy = y0 + r; if (iy < 0 || iy >= g.H) continue;
      const float4* row = x + ((long long)b * g.H + iy) * g.W * C4 + c;
      for (int s = 0; s < g.kw; ++s) {
        const int ix = x0 + s; if (ix < 0 || ix >= g.W) continue;
        const float4 v = row[(long long)ix * C4];
        if (AVG) { a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
        else { if (v.x > a.x) a.x = v.x; if (v.y > a.y) a.y = v.y; if (v.z > a.z) a.z = v.z; if (v.w > a.w) a.w = v.w; }
      }
    }
    y[i] = AVG ? make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv) : a;
  }
}
// Global average pooling (one window = the whole image): a block takes one image and up to 32 channel groups; its 256
// threads are (position lanes) x (channel-group lanes), so a step reads whole contiguous rows of the image and every thread
// has only H*W / (position lanes) loads in a row; the position lanes are folded through shared memory.
__global__ void __launch_bounds__(NT) global_avgpool_v4_kernel(const float4* __restrict__ x, float4* __restrict__ y, int HW, int C4, int CL) {
  __shared__ float4 red[NT];
  const int PL = NT / CL, cl = threadIdx.x % CL, pl = threadIdx.x / CL;
  const int n = blockIdx.y, c = blockIdx.x * CL + cl;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  if (pl < PL && c < C4) {
    const float4* src = x + (long long)n * HW * C4 + c;
#pragma unroll 4
    for (int p = pl; p < HW; p += PL) { const float4 v = src[(long long)p * C4]; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
  }
  red[threadIdx.x] = a;
  __syncthreads();
  if (pl == 0 && c < C4) {
    for (int l = 1; l < PL; ++l) { const float4 v = red[l * CL + cl]; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
    const float inv = 1.f / (float)HW;
    y[(long long)n * C4 + c] = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
  }
}
// DIRECT (windows do not overlap): every window position is written with a plain store - dy at the first maximum, zero
// elsewhere; otherwise dy is added at the first maximum with an atomic (dx zeroed by the caller).
template <bool DIRECT>
__global__ void __launch_bounds__(NT) maxpool_bwd_v4_kernel(const float4* __restrict__ dy, const float4* __restrict__ x, float* __restrict__ dx,
                                                            PoolGeom g, int accum) {
  const unsigned C4 = (unsigned)g.C >> 2, n = (unsigned)g.N * g.P * g.Q * C4;
  for (unsigned i = blockIdx.x * NT + threadIdx.x; i < n; i += gridDim.x * NT) {
    const unsigned c = i % C4; unsigned t = i / C4; const int q = t % g.Q; t /= g.Q; const int p = t % g.P, b = t / g.P;
    const int y0 = p * g.sh - g.ph, x0 = q * g.sw - g.pw;
    float best[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};
    int arg[4] = {-1, -1, -1, -1};
    for (int r = 0; r < g.kh; ++r) {
      const int iy = y0 + r; if (iy < 0 || iy >= g.H) continue;
      const float4* row = x + ((long long)b * g.H + iy) * g.W * C4 + c;
      for (int s = 0; s < g.kw; ++s) {
        const int ix = x0 + s; if (ix < 0 || ix >= g.W) continue;
        const float4 v = row[(long long)ix * C4];
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) if (vv[e] > best[e]) { best[e] = vv[e]; arg[e] = r * g.kw + s; }
      }
    }
    const float4 g4 = dy[i];
    const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
    if (DIRECT) {
      for (int r = 0; r < g.kh; ++r) {
        const int iy = y0 + r; if (iy < 0 || iy >= g.H) continue;
        for (int s = 0; s < g.kw; ++s) {
          const int ix = x0 + s; if (ix < 0 || ix >= g.W) continue;
          float4* d = reinterpret_cast<float4*>(dx) + (((long long)b * g.H + iy) * g.W + ix) * C4 + c;
          const int tap = r * g.kw + s;
          float4 o = make_float4(arg[0] == tap ? gg[0] : 0.f, arg[1] == tap ? gg[1] : 0.f, arg[2] == tap ? gg[2] : 0.f, arg[3] == tap ? gg[3] : 0.f);
          if (accum) { const float4 old = *d; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
          *d = o;
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (arg[e] >= 0) {
          const int r = arg[e] / g.kw, s = arg[e] - r * g.kw;
          atomicAdd(dx + ((((long long)b * g.H + y0 + r) * g.W + x0 + s) * C4 + c) * 4 + e, gg[e]);
        }
    }
  }
}

// average pooling, divisor = kh*kw always (padding counted)
__global__ void avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, PoolGeom g) {
  long long n = (long long)g.N * g.P * g.Q * g.C;
  const float inv = 1.f / (float)(g.kh * g.kw);
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int c = (int)(i % g.C); long long t = i / g.C; int q = (int)(t % g.Q); t /= g.Q; int p = (int)(t % g.P); int b = (int)(t / g.P);
    float s = 0.f;
    for (int r = 0; r < g.kh; ++r) {
      int iy = p * g.sh - g.ph + r; if (iy < 0 || iy >= g.H) continue;
      for (int ss = 0; ss < g.kw; ++ss) {
        int ix = q * g.sw - g.pw + ss; if (ix < 0 || ix >= g.W) continue;
        s += x[(((long long)b * g.H + iy) * g.W + ix) * g.C + c];
      }
    }
    y[i] = s * inv;
  }
}
// gather form: each input element sums the windows that cover it (no atomics)
__global__ void avgpool_bwd_kernel(const float* __restrict__ dy, float* __restrict__ dx, PoolGeom g, int accum) {
  long long n = (long long)g.N * g.H * g.W * g.C;
  const float inv = 1.f / (float)(g.kh * g.kw);
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int c = (int)(i % g.C); long long t = i / g.C; int ix = (int)(t % g.W); t /= g.W; int iy = (int)(t % g.H); int b = (int)(t / g.H);
    float s = 0.f;
    for (int r = 0; r < g.kh; ++r) {
      int ty = iy + g.ph - r; if (ty < 0 || ty % g.sh) continue; int p = ty / g.sh; if (p >= g.P) continue;
      for (int ss = 0; ss < g.kw; ++ss) {
        int tx = ix + g.pw - ss; if (tx < 0 || tx % g.sw) continue; int q = tx / g.sw; if (q >= g.Q) continue;
        s += dy[(((long long)b * g.P + p) * g.Q + q) * g.C + c];
      }
    }
    dx[i] = accum ? dx[i] + s * inv : s * inv;
  }
}

// 16-byte form of the kernel above (C % 4 == 0): one thread = four channels of one input position
__global__ void __launch_bounds__(NT) avgpool_bwd_v4_kernel(const float4* __restrict__ dy, float4* __restrict__ dx, PoolGeom g, int accum) {
  const unsigned C4 = (unsigned)g.C >> 2, n = (unsigned)g.N * g.H * g.W * C4;
  const float inv = 1.f / (float)(g.kh * g.kw);
  for (unsigned i = blockIdx.x * NT + threadIdx.x; i < n; i += gridDim.x * NT) {
    const unsigned c = i % C4; unsigned t = i / C4; const int ix = t % g.W; t /= g.W; const int iy = t % g.H, b = t / g.H;
    float4 s = make_float4(0, 0, 0, 0);
    for (int r = 0; r < g.kh; ++r) {
      const int ty = iy + g.ph - r; if (ty < 0 || ty % g.sh) continue; const int p = ty / g.sh; if (p >= g.P) continue;
      for (int ss = 0; ss < g.kw; ++ss) {
        const int tx = ix + g.pw - ss; if (tx < 0 || tx % g.sw) continue; const int q = tx / g.sw; if (q >= g.Q) continue;
        const float4 v = dy[(((long long)b * g.P + p) * g.Q + q) * C4 + c];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    float4 o = make_float4(s.x * inv, s.y * inv, s.z * inv, s.w * inv);
    if (accum) { const float4 d = dx[i]; o.x += d.x; o.y += d.y; o.z += d.z; o.w += d.w; }
    dx[i] = o;
  }
}

// across-channel LRN (Caffe): y = x * (k + alpha/size * sum_{window} x^2)^-beta
__global__ void lrn_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ scale, long long M, int C, int size, float alpha, float beta, float k) {
  long long n = M * C; int half = size / 2;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    long long m = i / C; int c = (int)(i % C);
    float s = 0.f;
    for (int j = max(0, c - half); j <= min(C - 1, c + half); ++j) { float v = x[m * C + j]; s += v * v; }
    float sc = k + alpha / size * s;
    scale[i] = sc;
    y[i] = x[i] * __powf(sc, -beta);
  }
}
__global__ void lrn_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ scale,
                               float* __restrict__ dx, long long M, int C, int size, float alpha, float beta, int accum) {
  long long n = M * C; int half = size / 2;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    long long m = i / C; int c = (int)(i % C);
    float s = 0.f;
    for (int j = max(0, c - half); j <= min(C - 1, c + half); ++j) s += dy[m * C + j] * y[m * C + j] / scale[m * C + j];
    float o = dy[i] * __powf(scale[i], -beta) - 2.f * alpha * beta / size * x[i] * s;
    dx[i] = accum ? dx[i] + o : o;
  }
}

// Input transform: NCHW source -> channels-last destination with crop / mirror / mean / scale.
// Per example three Philox words (counter = example): crop row, crop column, mirror bit.
struct TransformArgs { int N, C, H, W, OH, OW; int mirror; int training; float scale; int mean_mode; /*0 none,1 per channel,2 per pixel (full image)*/ unsigned stream; };
__global__ void transform_kernel(const float* __restrict__ src, float* __restrict__ dst, const float* __restrict__ mean, TransformArgs a,
                                 const XbTaskParams* __restrict__ tp) {
  long long n = (long long)a.N * a.OH * a.OW * a.C;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int c = (int)(i % a.C); long long t = i / a.C; int ox = (int)(t % a.OW); t /= a.OW; int oy = (int)(t % a.OH); int b = (int)(t / a.OH);
    int ho = (a.H - a.OH) / 2, wo = (a.W - a.OW) / 2; bool flip = false;
    if (a.training) {
      // example b uses elements 3b, 3b+1, 3b+2 of the stream
      uint32_t r[3];
#pragma unroll
      for (int e = 0; e < 3; ++e) {
        uint32_t idx = 3u * b + e;
        uint4 w = xb_philox4x32(idx >> 2, tp->task_id, a.stream, 0u, tp->seed_lo, tp->seed_hi);
        uint32_t lanes[4] = {w.x, w.y, w.z, w.w};
        r[e] = lanes[idx & 3u];
      }
      ho = (int)(r[0] % (uint32_t)(a.H - a.OH + 1));
      wo = (int)(r[1] % (uint32_t)(a.W - a.OW + 1));
      flip = a.mirror && (r[2] & 1u);
    }
    int sx = flip ? (a.OW - 1 - ox) : ox;
    int iy = oy + ho, ix = sx + wo;
    float v = src[(((long long)b * a.C + c) * a.H + iy) * a.W + ix];
    if (a.mean_mode == 1) v -= mean[c];
    else if (a.mean_mode == 2) v -= mean[((long long)c * a.H + iy) * a.W + ix];
    dst[i] = v * a.scale;
  }
}
// channels-last -> NCHW (used to hand activations back in the public layout)
__global__ void nhwc_to_nchw_kernel(const float* __restrict__ src, float* __restrict__ dst, int N, int C, int H, int W) {
  long long n = (long long)N * C * H * W;
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n; i += (long long)gridDim.x * NT) {
    int x = (int)(i % W); long long t = i / W; int y = (int)(t % H); t /= H; int c = (int)(t % C); int b = (int)(t / C);
    dst[i] = src[(((long long)b * H + y) * W + x) * C + c];
  }
}
// column sums: out[c] += sum_m a[m][c]  (bias gradients)
__global__ void colsum_kernel(const float* __restrict__ a, float* __restrict__ out, int M, int C, int rows_per_block) {
  int r0 = blockIdx.x * rows_per_block, r1 = min(M, r0 + rows_per_block);
  for (int c = threadIdx.x; c < C; c += NT) {
    float s = 0.f;
    for (int r = r0; r < r1; ++r) s += a[(long long)r * C + c];
    atomicAdd(&out[c], s);
  }
}
// the same for C % 4 == 0, C <= 1024: the block's 256 threads form (256 / C4) row lanes x C4 column groups, every thread
// adds 16-byte loads of its rows four at a time, the row lanes are folded through shared memory, one atomic per column
__global__ void __launch_bounds__(NT) colsum_v4_kernel(const float4* __restrict__ a, float* __restrict__ out, int M, int C4, int rows_per_block) {
  __shared__ float4 red[NT];
  const int lanes = NT / C4, cg = threadIdx.x % C4, lane = threadIdx.x / C4;
  const int r0 = blockIdx.x * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float4 s = make_float4(0, 0, 0, 0);
  if (lane < lanes) {
    int r = r0 + lane;
    for (; r + 3 * lanes < r1; r += 4 * lanes) {
      const float4 v0 = a[(long long)r * C4 + cg], v1 = a[(long long)(r + lanes) * C4 + cg], v2 = a[(long long)(r + 2 * lanes) * C4 + cg],
                   v3 = a[(long long)(r + 3 * lanes) * C4 + cg];
      s.x += (v0.x + v1.x) + (v2.x + v3.x); s.y += (v0.y + v1.y) + (v2.y + v3.y); s.z += (v0.z + v1.z) + (v2.z + v3.z); s.w += (v0.w + v1.w) + (v2.w + v3.w);
    }
    for (; r < r1; r += lanes) { const float4 v = a[(long long)r * C4 + cg]; s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
  }
  red[threadIdx.x] = s;
  __syncthreads();
  if (lane == 0) {
    for (int l = 1; l < lanes; ++l) { const float4 v = red[l * C4 + cg]; s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w; }
    atomicAdd(out + 4 * cg, s.x); atomicAdd(out + 4 * cg + 1, s.y); atomicAdd(out + 4 * cg + 2, s.z); atomicAdd(out + 4 * cg + 3, s.w);
  }
}
}  // namespace

XB_API int xb_act_forward(const float* x, float* y, long long n, int mode, float slope, float ceiling, cudaStream_t st) {
  if (n % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0)
    act_fwd_v4_kernel<<<grid_for(n / 4, 2), NT, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), n / 4, mode, slope, ceiling);
  else
    act_fwd_kernel<<<grid_for(n, 4), NT, 0, st>>>(x, y, n, mode, slope, ceiling);
  return (int)cudaGetLastError();
}
XB_API int xb_act_backward(const float* dy, const float* x, const float* y, float* dx, long long n, int mode, float slope, float ceiling,
                           int accum, cudaStream_t st) {
  if (n % 4 == 0 && ((uintptr_t)dy % 16) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)dx % 16) == 0)
    act_bwd_v4_kernel<<<grid_for(n / 4, 2), NT, 0, st>>>(reinterpret_cast<const float4*>(dy), reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(y),
                                                        reinterpret_cast<float4*>(dx), n / 4, mode, slope, ceiling, accum);
  else
    act_bwd_kernel<<<grid_for(n, 4), NT, 0, st>>>(dy, x, y, dx, n, mode, slope, ceiling, accum);
  return (int)cudaGetLastError();
}
XB_API int xb_weighted_sum(const float* const* xs, const float* coef, int n_in, float* y, long long n, int accum, cudaStream_t st) {
  if (n_in < 1 || n_in > 4) return -XB_BAD_ARG;
  SumArgs a; a.n_in = n_in;
  bool aligned = ((uintptr_t)y % 16) == 0;
  for (int i = 0; i < 4; ++i) { a.x[i] = i < n_in ? xs[i] : nullptr; a.coef[i] = i < n_in ? coef[i] : 0.f; if (i < n_in && ((uintptr_t)xs[i] % 16)) aligned = false; }
  long long n4 = aligned ? n / 4 : 0;
  long long work = n4 > (n - n4 * 4) ? n4 : (n - n4 * 4);
  int blocks = grid_for(work);
  weighted_sum_kernel<<<blocks, NT, 0, st>>>(a, y, n4, n, accum);
  return (int)cudaGetLastError();
}
XB_API int xb_dropout(const float* x, float* y, long long n, float ratio, unsigned stream, const XbTaskParams* tp, int accum, cudaStream_t st) {
  const bool vec = ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0;
  dropout_kernel<<<grid_for((n + 3) / 4, 2), NT, 0, st>>>(x, y, n, ratio, stream, tp, accum, vec);
  return (int)cudaGetLastError();
}
XB_API int xb_concat_copy(const float* src, float* dst, long long M, int Cs, int Ct, int coff, int to_wide, int accum, cudaStream_t st) {
  concat_copy_kernel<<<grid_for(M * Cs, 2), NT, 0, st>>>(src, dst, M, Cs, Ct, coff, to_wide, accum);
  return (int)cudaGetLastError();
}
static inline bool pool_vec_ok(const PoolGeom& g, const void* a, const void* b) {
  return (g.C % 4) == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 && (long long)g.N * g.P * g.Q * (g.C / 4) < (1ll << 31) &&
         (long long)g.N * g.H * g.W < (1ll << 31);
}
XB_API int xb_pool_forward(const float* x, float* y, const int* geom12, int average, cudaStream_t st) {
  PoolGeom g; memcpy(&g, geom12, sizeof(g));
  long long n = (long long)g.N * g.P * g.Q * g.C;
  if (average && pool_vec_ok(g, x, y) && g.P == 1 && g.Q == 1 && g.kh == g.H && g.kw == g.W && g.ph == 0 && g.pw == 0) {
    const int C4 = g.C / 4;
    int CL = 1; while (CL < 32 && CL < C4) CL <<= 1;         // channel-group lanes: a power of two <= 32
    dim3 grid((unsigned)((C4 + CL - 1) / CL), (unsigned)g.N);
    global_avgpool_v4_kernel<<<grid, NT, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), g.H * g.W, C4, CL);
    return (int)cudaGetLastError();
  }
  if (pool_vec_ok(g, x, y)) {
    if (average) pool_fwd_v4_kernel<true><<<grid_for(n / 4), NT, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), g);
    else pool_fwd_v4_kernel<false><<<grid_for(n / 4), NT, 0, st>>>(reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), g);
  } else if (average) avgpool_fwd_kernel<<<grid_for(n), NT, 0, st>>>(x, y, g);
  else maxpool_fwd_kernel<<<grid_for(n), NT, 0, st>>>(x, y, g);
  return (int)cudaGetLastError();
}
// max: dx must be pre-zeroed unless accumulating (scatter with atomics); average: gather form
XB_API int xb_pool_backward(const float* dy, const float* x, float* dx, const int* geom12, int average, int accum, cudaStream_t st) {
  PoolGeom g; memcpy(&g, geom12, sizeof(g));
  if (average) {
    if (pool_vec_ok(g, dy, dx) && (long long)g.N * g.H * g.W * (g.C / 4) < (1ll << 31))
      avgpool_bwd_v4_kernel<<<grid_for((long long)g.N * g.H * g.W * (g.C / 4)), NT, 0, st>>>(reinterpret_cast<const float4*>(dy), reinterpret_cast<float4*>(dx), g, accum);
    else
      avgpool_bwd_kernel<<<grid_for((long long)g.N * g.H * g.W * g.C), NT, 0, st>>>(dy, dx, g, accum);
  } else {
    const long long n = (long long)g.N * g.P * g.Q * g.C;
    const bool vec = pool_vec_ok(g, x, dy) && ((uintptr_t)dx % 16) == 0;
    const bool disjoint = g.kh <= g.sh && g.kw <= g.sw;                       // a position belongs to at most one window
    const bool covered = disjoint && g.kh == g.sh && g.kw == g.sw && g.ph == 0 && g.pw == 0 && (long long)g.P * g.sh >= g.H && (long long)g.Q * g.sw >= g.W;
    if (!accum && !(vec && covered)) { cudaError_t e = cudaMemsetAsync(dx, 0, sizeof(float) * (size_t)g.N * g.H * g.W * g.C, st); if (e != cudaSuccess) return (int)e; }
    if (vec && disjoint)
      maxpool_bwd_v4_kernel<true><<<grid_for(n / 4), NT, 0, st>>>(reinterpret_cast<const float4*>(dy), reinterpret_cast<const float4*>(x), dx, g, accum);
    else if (vec)
      maxpool_bwd_v4_kernel<false><<<grid_for(n / 4), NT, 0, st>>>(reinterpret_cast<const float4*>(dy), reinterpret_cast<const float4*>(x), dx, g, accum);
    else
      maxpool_bwd_kernel<<<grid_for(n), NT, 0, st>>>(dy, x, dx, g);
  }
  return (int)cudaGetLastError();
}
XB_API int xb_lrn_forward(const float* x, float* y, float* scale, long long M, int C, int size, float alpha, float beta, float k, cudaStream_t st) {
  lrn_fwd_kernel<<<grid_for(M * C), NT, 0, st>>>(x, y, scale, M, C, size, alpha, beta, k);
  return (int)cudaGetLastError();
}
XB_API int xb_lrn_backward(const float* dy, const float* x, const float* y, const float* scale, float* dx, long long M, int C, int size,
                           float alpha, float beta, int accum, cudaStream_t st) {
  lrn_bwd_kernel<<<grid_for(M * C), NT, 0, st>>>(dy, x, y, scale, dx, M, C, size, alpha, beta, accum);
  return (int)cudaGetLastError();
}
XB_API int xb_transform(const float* src, float* dst, const float* mean, int N, int C, int H, int W, int OH, int OW, int mirror, int training,
                        float scale, int mean_mode, unsigned stream, const XbTaskParams* tp, cudaStream_t st) {
  TransformArgs a{N, C, H, W, OH, OW, mirror, training, scale, mean_mode, stream};
  transform_kernel<<<grid_for((long long)N * OH * OW * C), NT, 0, st>>>(src, dst, mean, a, tp);
  return (int)cudaGetLastError();
}
XB_API int xb_nhwc_to_nchw(const float* src, float* dst, int N, int C, int H, int W, cudaStream_t st) {
  nhwc_to_nchw_kernel<<<grid_for((long long)N * C * H * W), NT, 0, st>>>(src, dst, N, C, H, W);
  return (int)cudaGetLastError();
}
XB_API int xb_colsum(const float* a, float* out, int M, int C, cudaStream_t st) {
  if (C % 4 == 0 && C <= 4 * NT && ((uintptr_t)a % 16) == 0 && M >= 64) {
    const int C4 = C / 4, lanes = NT / C4;
    int rpb = xb_ceil_div(M, 296); if (rpb < lanes * 8) rpb = lanes * 8;
    colsum_v4_kernel<<<xb_ceil_div(M, rpb), NT, 0, st>>>(reinterpret_cast<const float4*>(a), out, M, C4, rpb);
    return (int)cudaGetLastError();
  }
  int rpb = xb_ceil_div(M, 148); if (rpb < 32) rpb = 32;
  colsum_kernel<<<xb_ceil_div(M, rpb), NT, 0, st>>>(a, out, M, C, rpb);
  return (int)cudaGetLastError();
}

// ---- busy-wait for a number of SM clock cycles (kernels/sleep.cu:4-23; used to measure a pipeline's makespan) --------------
// Bounded: at most 2^31 cycles (about a second), so a wrong argument cannot park a GPU.
namespace {
__global__ void sleep_kernel(long long cycles) {
  const long long t0 = clock64();
  while (clock64() - t0 < cycles) { }
}
}  // namespace
XB_API int xb_sleep(long long cycles, cudaStream_t st) {
  if (cycles < 0) return -XB_BAD_ARG;
  if (cycles > (1ll << 31)) cycles = 1ll << 31;
  sleep_kernel<<<1, 1, 0, st>>>(cycles);
  return (int)cudaGetLastError();
}
