// Image pre-processing of the record pipeline on the GPU: crop, horizontal flip, bilinear resize, scaling to [-1, 1]
// and interleaved-to-planar conversion of DECODED images, one launch per batch.
//
// The reference does this on the CPU, per image, after libjpeg (clib-multigpu/image/image.c:255-302 crop, :304-334 flip,
// :692-824 bilinear resize, image/recordreader.c:448-560 scale x/127.5 - 1 and HWC -> CHW).  The host runtime has the
// same CPU path (csrc/data/record.cpp); this kernel is its device twin for pipelines that upload the decoded bytes
// (3 bytes per pixel) instead of the finished example (12 bytes per output pixel) and leave the arithmetic to the GPU.
// The arithmetic is written with explicitly rounded single operations (no fused multiply-add, IEEE division), in the
// CPU path's order, so both paths produce bit-identical examples from the same crop plan.
#include "common.cuh"

// One image of the batch: where its interleaved RGB bytes start in the packed buffer, its size, the crop window and flip.
struct XbImageDesc {
  long long offset;
  int W, H;
  int x0, y0, cw, ch;
  int flip;
  int pad;
};

namespace {

__global__ void __launch_bounds__(256) image_crop_resize_kernel(const uint8_t* __restrict__ rgb, const XbImageDesc* __restrict__ descs,
                                                                 float* __restrict__ out, int S) {
  const XbImageDesc d = descs[blockIdx.y];
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= S * S) return;
  const int oy = p / S, ox = p - oy * S;
  const float sx = __fdiv_rn((float)d.cw, (float)S), sy = __fdiv_rn((float)d.ch, (float)S);
  const float fy = __fmul_rn((float)oy, sy);
  const int iy = (int)fy;
  const float wy = __fsub_rn(fy, (float)iy);
  const int iy1 = min(iy + 1, d.ch - 1);
  const int sxp = d.flip ? (S - 1 - ox) : ox;
  const float fx = __fmul_rn((float)sxp, sx);
  const int ix = (int)fx;
  const float wx = __fsub_rn(fx, (float)ix);
  const int ix1 = min(ix + 1, d.cw - 1);
  const uint8_t* img = rgb + d.offset;
  const uint8_t* p00 = img + ((size_t)(d.y0 + iy) * d.W + d.x0 + ix) * 3;
  const uint8_t* p01 = img + ((size_t)(d.y0 + iy) * d.W + d.x0 + ix1) * 3;
  const uint8_t* p10 = img + ((size_t)(d.y0 + iy1) * d.W + d.x0 + ix) * 3;
  const uint8_t* p11 = img + ((size_t)(d.y0 + iy1) * d.W + d.x0 + ix1) * 3;
  const float inv = __fdiv_rn(1.f, 127.5f);
  float* o = out + (size_t)blockIdx.y * 3 * S * S + p;
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float a = (float)p00[c], b = (float)p10[c];
    const float top = __fadd_rn(a, __fmul_rn((float)((int)p01[c] - (int)p00[c]), wx));
    const float bot = __fadd_rn(b, __fmul_rn((float)((int)p11[c] - (int)p10[c]), wx));
    const float v = __fadd_rn(top, __fmul_rn(__fsub_rn(bot, top), wy));
    o[(size_t)c * S * S] = __fsub_rn(__fmul_rn(v, inv), 1.f);
  }
}

}  // namespace

XB_API int xb_image_desc_size() { return (int)sizeof(XbImageDesc); }

// rgb: packed decoded images (device), descs: n descriptors (device), out: n x 3 x S x S floats (device).
// Every crop window must lie inside its image (checked by the caller that builds the plan).
XB_API int xb_image_crop_resize(const uint8_t* rgb, const XbImageDesc* descs, int n, int S, float* out, cudaStream_t st) {
  if (n <= 0 || S <= 0) return -XB_BAD_ARG;
  dim3 grid((S * S + 255) / 256, n);
  image_crop_resize_kernel<<<grid, 256, 0, st>>>(rgb, descs, out, S);
  return (int)cudaGetLastError();
}
