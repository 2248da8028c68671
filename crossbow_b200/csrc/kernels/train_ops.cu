// Loss / accuracy head and the per-task local optimiser.
//
// softmax + cross-entropy + accuracy + (p - onehot)/N in ONE kernel replaces cudnnSoftmaxForward, the hand-written
// loss / loss-gradient / accuracy kernels and their cuBLAS sscal/sasum reductions
// (clib-multigpu/kernels/cudnnsoftmax.cu, softmaxloss.cu:3-27,117-144, softmaxlossgradient.cu:5-34,128-131,
// accuracy.cu:3-30,73-76); loss and accuracy land directly in a host-mapped result slot.
// The fused optimiser replaces the 4-6 cuBLAS level-1 passes per task of kernels/optimisers/{sma,default,
// synchronoussgd}.cu with a single pass over the flat parameter vector.
#include "common.cuh"
#include <float.h>

namespace {

// One warp per example row; one block per launch (batch sizes here are <= a few thousand rows).
// mode: 0 BATCH / FULL (divide by rows), 1 VALID (divide by non-ignored rows), 2 NONE
__global__ void __launch_bounds__(1024) softmax_xent_kernel(const float* __restrict__ logits, const int* __restrict__ labels,
                                                            float* __restrict__ probs, float* __restrict__ dlogits,
                                                            float* __restrict__ result /* [0]=loss [1]=accuracy */,
                                                            int rows, int classes, int ignore_label, int mode, int part, int parts) {
  __shared__ float s_loss[32], s_acc[32], s_valid[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float loss_sum = 0.f, acc_sum = 0.f, valid_sum = 0.f;
  for (int r = warp; r < rows; r += nwarps) {
    const float* x = logits + (long long)r * classes;
    float mx = -FLT_MAX; int arg = 0;
    for (int c = lane; c < classes; c += 32) { float v = x[c]; if (v > mx) { mx = v; arg = c; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, mx, o); int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (om > mx || (om == mx && oa < arg)) { mx = om; arg = oa; }
    }
    float se = 0.f;
    for (int c = lane; c < classes; c += 32) se += __expf(x[c] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    const float inv = 1.f / se;
    const int label = labels[r];
    const bool valid = label != ignore_label;
    for (int c = lane; c < classes; c += 32) {
      float p = __expf(x[c] - mx) * inv;
      if (probs) probs[(long long)r * classes + c] = p;
      if (dlogits) dlogits[(long long)r * classes + c] = valid ? (p - (c == label ? 1.f : 0.f)) : 0.f;   // scaled below
    }
    if (lane == 0) {
      if (valid) {
        float pl = __expf(x[label] - mx) * inv;
        loss_sum += -__logf(fmaxf(pl, FLT_MIN));
        valid_sum += 1.f;
      }
      acc_sum += (arg == label) ? 1.f : 0.f;
    }
  }
  if (lane == 0) { s_loss[warp] = loss_sum; s_acc[warp] = acc_sum; s_valid[warp] = valid_sum; }
  __syncthreads();
  float denom;
  {
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v += s_valid[w];
    denom = (mode == 1) ? fmaxf(v, 1.f) : (mode == 2 ? 1.f : (float)rows);
  }
  if (threadIdx.x == 0) {
    float l = 0.f, a = 0.f;
    for (int w = 0; w < nwarps; ++w) { l += s_loss[w]; a += s_acc[w]; }
    // part p of `parts` sub-batches of one task: the slot ends up holding the mean over the parts
    const float wgt = 1.f / (float)parts;
    result[0] = (part ? result[0] : 0.f) + wgt * l / denom;
    result[1] = (part ? result[1] : 0.f) + wgt * a / (float)rows;
  }
  if (dlogits) {
    __syncthreads();
    const float sc = 1.f / denom;
    for (long long i = threadIdx.x; i < (long long)rows * classes; i += blockDim.x) dlogits[i] *= sc;
  }
}

// argmax per row as float (classify.cu:3-26)
__global__ void classify_kernel(const float* __restrict__ x, float* __restrict__ out, int rows, int classes) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float mx = -FLT_MAX; int arg = 0;
  for (int c = 0; c < classes; ++c) { float v = x[(long long)r * classes + c]; if (v > mx) { mx = v; arg = c; } }
  out[r] = (float)arg;
}

// sum of squares of the gradient -> norm2[0] (must be zeroed before)
__global__ void sumsq_kernel(const float* __restrict__ g, float* __restrict__ norm2, long long n) {
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) { float v = g[i]; s += v * v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float sh[32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[w]; atomicAdd(norm2, t); }
}

// update_mode: 0 = local step (SMA / EAMSGD / Polyak-Ruppert), 1 = local step + same step applied to z (DEFAULT),
//              2 = accumulate -lr*g into the device gradient accumulator, weights untouched (synchronous SGD)
struct OptArgs {
  float* w; float* g; float* last; float* prev; float* z_or_gacc; const float* lr_mult; const float* norm2;
  const XbTaskParams* tp; long long n4; int update_mode;
};
__global__ void __launch_bounds__(256) fused_optimiser_kernel(OptArgs a) {
  const XbTaskParams tp = *a.tp;
  float gscale = 1.f;
  if (tp.clip >= 0.f && a.norm2) { float l2 = sqrtf(*a.norm2); if (l2 > tp.clip) gscale = tp.clip / l2; }
  // Four float4 lanes per thread and step, all loads ahead of the first store: the compiler may not hoist loads above
  // stores to pointers that could alias, and a one-lane loop leaves most of the memory pipeline idle.
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * 256;
  for (long long i0 = blockIdx.x * 256LL + threadIdx.x; i0 < a.n4; i0 += U * stride) {
    float4 w[U], g[U], l[U], m[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) ok[u] = i0 + u * stride < a.n4;
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) { w[u] = reinterpret_cast<float4*>(a.w)[i0 + u * stride]; g[u] = reinterpret_cast<float4*>(a.g)[i0 + u * stride]; }
    if (a.update_mode != 2 && tp.momentum > 0.f) {
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) l[u] = reinterpret_cast<float4*>(a.last)[i0 + u * stride];
    }
    if (a.lr_mult) {
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) m[u] = reinterpret_cast<const float4*>(a.lr_mult)[i0 + u * stride];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!ok[u]) continue;
      const long long i = i0 + u * stride;
      reinterpret_cast<float4*>(a.g)[i] = make_float4(0, 0, 0, 0);     // the next task's wgrad accumulates from zero
      float wv[4] = {w[u].x, w[u].y, w[u].z, w[u].w}, gv[4] = {g[u].x, g[u].y, g[u].z, g[u].w}, lm[4] = {1.f, 1.f, 1.f, 1.f};
      if (a.lr_mult) { lm[0] = m[u].x; lm[1] = m[u].y; lm[2] = m[u].z; lm[3] = m[u].w; }
      float step[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float gg = gv[e] * gscale;
        if (tp.weight_decay > 0.f) gg += tp.weight_decay * (tp.l1 ? (wv[e] > 0.f ? 1.f : (wv[e] < 0.f ? -1.f : 0.f)) : wv[e]);
        step[e] = -tp.lr * lm[e] * gg;
      }
      if (a.update_mode == 2) {
        float* acc = a.z_or_gacc + i * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) atomicAdd(acc + e, step[e]);       // several replicas of the device accumulate concurrently
        continue;
      }
      reinterpret_cast<float4*>(a.prev)[i] = w[u];                      // snapshot BEFORE the step
      if (tp.momentum > 0.f) {
        float lv[4] = {l[u].x, l[u].y, l[u].z, l[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float s = step[e] + tp.momentum * lv[e];
          lv[e] = s;
          step[e] = tp.nesterov ? (step[e] + tp.momentum * s) : s;
        }
        reinterpret_cast<float4*>(a.last)[i] = make_float4(lv[0], lv[1], lv[2], lv[3]);
      }
      reinterpret_cast<float4*>(a.w)[i] = make_float4(wv[0] + step[0], wv[1] + step[1], wv[2] + step[2], wv[3] + step[3]);
      if (a.update_mode == 1) {
        float* z = a.z_or_gacc + i * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) atomicAdd(z + e, step[e]);
      }
    }
  }
}
// Matrix factorisation (clib-multigpu/kernels/matfact.cu:6-61): one warp per (row, column, rating) example.
//   pred = <U[row], V[col]> ; err = rating - pred
//   loss = (sum err^2 + lambda * (sum |U[row]|^2 + sum |V[col]|^2)) / batch        -> result[0]
//   dU[row] += (-2 err V[col] + 2 lambda U[row]) / batch ; dV[col] likewise (atomics: rows repeat within a batch)
__global__ void matfact_kernel(const float* __restrict__ triples, int stride, const int* __restrict__ ratings_i, const float* __restrict__ U,
                               const float* __restrict__ V, float* __restrict__ dU, float* __restrict__ dV, float* __restrict__ result,
                               int batch, int latents, float lambda, int rows, int cols) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= batch) return;
  const float* t = triples + (long long)warp * stride;
  const int r = min(max((int)t[0], 0), rows - 1), c = min(max((int)t[1], 0), cols - 1);
  const float rating = ratings_i ? (float)ratings_i[warp] : t[2];
  const float* u = U + (long long)r * latents; const float* v = V + (long long)c * latents;
  float dot = 0.f, nu = 0.f, nv = 0.f;
  for (int k = lane; k < latents; k += 32) { float a = u[k], b = v[k]; dot += a * b; nu += a * a; nv += b * b; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { dot += __shfl_xor_sync(0xffffffffu, dot, o); nu += __shfl_xor_sync(0xffffffffu, nu, o); nv += __shfl_xor_sync(0xffffffffu, nv, o); }
  const float err = rating - dot, inv = 1.f / (float)batch;
  if (dU)
    for (int k = lane; k < latents; k += 32) {
      float a = u[k], b = v[k];
      atomicAdd(&dU[(long long)r * latents + k], (-2.f * err * b + 2.f * lambda * a) * inv);
      atomicAdd(&dV[(long long)c * latents + k], (-2.f * err * a + 2.f * lambda * b) * inv);
    }
  if (lane == 0) atomicAdd(&result[0], (err * err + lambda * (nu + nv)) * inv);
}
}  // namespace

// result[0] must be zero on entry (it is accumulated); result[1] (accuracy) is set to 0.
XB_API int xb_matfact(const float* triples, int stride, const int* ratings, const float* U, const float* V, float* dU, float* dV, float* result,
                      int batch, int latents, float lambda, int rows, int cols, cudaStream_t st) {
  XB_CUDA_CHECK(cudaMemsetAsync(result, 0, 2 * sizeof(float), st));
  int threads = 256, blocks = xb_ceil_div((long long)batch * 32, threads);
  matfact_kernel<<<blocks, threads, 0, st>>>(triples, stride, ratings, U, V, dU, dV, result, batch, latents, lambda, rows, cols);
  return (int)cudaGetLastError();
}

XB_API int xb_softmax_xent(const float* logits, const int* labels, float* probs, float* dlogits, float* result, int rows, int classes,
                           int ignore_label, int mode, int part, int parts, cudaStream_t st) {
  int threads = rows * 32; if (threads > 1024) threads = 1024; if (threads < 32) threads = 32;
  softmax_xent_kernel<<<1, threads, 0, st>>>(logits, labels, probs, dlogits, result, rows, classes, ignore_label, mode, part, parts > 0 ? parts : 1);
  return (int)cudaGetLastError();
}
XB_API int xb_classify(const float* x, float* out, int rows, int classes, cudaStream_t st) {
  classify_kernel<<<xb_ceil_div(rows, 128), 128, 0, st>>>(x, out, rows, classes);
  return (int)cudaGetLastError();
}
XB_API int xb_grad_sumsq(const float* g, float* norm2, long long n, cudaStream_t st) {
  XB_CUDA_CHECK(cudaMemsetAsync(norm2, 0, sizeof(float), st));
  int blocks = (int)((n + 1023) / 1024); if (blocks > 592) blocks = 592; if (blocks < 1) blocks = 1;
  sumsq_kernel<<<blocks, 256, 0, st>>>(g, norm2, n);
  return (int)cudaGetLastError();
}
// 1: the kernels of a task's critical path are launched with programmatic stream serialisation (see common.cuh).
// ResNet-32, batch 64, one GPU: 48.7 K -> 53.2 K images/s with one replica, 78.2 K -> 86.7 K with two, 117.1 K -> 117.8 K
// with four (the other replicas already fill the gaps there), 132.8 K -> 135.6 K with eight; ResNet-50 +0.6 %.
int g_xb_pdl = 1;
XB_API void xb_set_pdl(int on) { g_xb_pdl = on ? 1 : 0; }
XB_API int xb_get_pdl() { return g_xb_pdl; }
static int g_opt_blocks = 148 * 4;
XB_API void xb_optimiser_set_blocks(int n) { g_opt_blocks = n > 0 ? n : 148 * 4; }
XB_API int xb_fused_optimiser(float* w, float* g, float* last, float* prev, float* z_or_gacc, const float* lr_mult, const float* norm2,
                              const XbTaskParams* tp, long long n, int update_mode, cudaStream_t st) {
  if (n % 4) return -XB_BAD_ARG;
  OptArgs a{w, g, last, prev, z_or_gacc, lr_mult, norm2, tp, n / 4, update_mode};
  // four 16-byte lanes per thread: small vectors get few, fully used blocks (0.46 M elements: 6.1 us with 148 blocks, 9.4 us with 592)
  int blocks = (int)((a.n4 + 1023) / 1024); if (blocks > g_opt_blocks) blocks = g_opt_blocks; if (blocks < 1) blocks = 1;
  fused_optimiser_kernel<<<blocks, 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}
