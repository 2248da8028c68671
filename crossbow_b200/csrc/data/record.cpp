// Record files + JPEG decoding + ImageNet-style augmentation + the pinned double buffer that feeds the learners.
//
// Record file (clib-multigpu/image/recordfile.c:175-362, scripts/datasets/imagenet/parse-records.py):
//   int32 count, then per record: int32 length (bytes that follow), int32 label, int32 nboxes,
//   float32 xmin[nboxes], ymin[nboxes], xmax[nboxes], ymax[nboxes], int32 height, int32 width, JPEG bytes.
// Pre-processing (image/image.c:255-334,692-975, image/recordreader.c:448-560):
//   train: sample a distorted bounding box (covers >= 10% of a labelled box, aspect ratio in [0.75, 1.33], area in
//          [5%, 100%] of the image, up to 100 attempts, else the whole image), crop, random horizontal flip, bilinear
//          resize to SxS, scale to [-1, 1] (x/127.5 - 1), interleaved HWC -> planar CHW;
//   test : aspect-preserving resize so that the shorter side is 1.145*S, centre crop SxS, same scaling.
// The reference links libjpeg; this file carries its own Huffman JPEG decoder instead: sequential and progressive
// frames, grey-scale / YCbCr / RGB / CMYK / YCCK, sampling factors up to 4 (triangle-filter chroma up-sampling for
// 2:1), restart intervals.  Arithmetic-coded, lossless and 12-bit files are reported as unsupported (the caller
// substitutes a grey image and counts the failure).
// Double buffer (clib-multigpu/doublebuffer.c, recorddataset.c): two halves of NB batches each; worker threads decode
// into the idle half while tasks consume the other; a swap waits (bounded) for the refill and for the tasks in flight.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

#include "../runtime/queues.hpp"

#define RT_API extern "C" __attribute__((visibility("default")))

namespace xb {

// ---------------------------------------------------------------------------------------------------------------------
// JPEG decoder: Huffman-coded baseline / extended sequential (SOF0, SOF1) and progressive (SOF2) files, 8-bit samples,
// 1 component (grey), 3 (YCbCr, or RGB when an Adobe marker says so) or 4 (CMYK / YCCK, converted to RGB as the
// reference does after libjpeg, image/image.c:119-139).  Every scan is decoded into a per-component coefficient array;
// de-quantisation, the inverse DCT, chroma up-sampling and colour conversion run once, after the last scan.
// The input is untrusted: table selectors, code lengths, run lengths and segment sizes are all checked.
// ---------------------------------------------------------------------------------------------------------------------
struct Huff { uint8_t bits[17]; uint8_t vals[256]; int mincode[17], maxcode[18], valptr[17]; bool set = false; };
struct Comp {
  int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0;
  int dc_pred = 0;
  int bw = 0, bh = 0;                // blocks per row / column of the coefficient array (padded to whole MCUs)
  int cw = 0, ch = 0;                // samples per row / column that belong to the image
  std::vector<int16_t> coef;         // bw * bh blocks of 64 coefficients, natural (row-major) order
  std::vector<uint8_t> plane; int pw = 0, ph = 0;
};

static const int kZigzag[64] = {0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6, 7, 14, 21, 28,
                                35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

struct BitReader {
  const uint8_t* p; const uint8_t* end; uint32_t buf = 0; int cnt = 0; bool marker = false;
  int bit() {
    if (cnt == 0) {
      if (p >= end) { marker = true; return 0; }
      uint8_t b = *p++;
      if (b == 0xFF) {
        if (p < end && *p == 0x00) ++p;
        else { marker = true; --p; return 0; }       // a marker: stop feeding bits
      }
      buf = b; cnt = 8;
    }
    --cnt;
    return (buf >> cnt) & 1;
  }
  int bits(int n) { int v = 0; while (n-- > 0) v = (v << 1) | bit(); return v; }
  void reset() { cnt = 0; marker = false; }
};

static void build_huff(Huff& h) {
  int code = 0, k = 0;
  for (int l = 1; l <= 16; ++l) {
    h.valptr[l] = k; h.mincode[l] = code;
    code += h.bits[l]; k += h.bits[l];
    h.maxcode[l] = h.bits[l] ? code - 1 : -1;
    code <<= 1;
  }
  h.maxcode[17] = 0x7fffffff; h.set = true;
}
static int decode_huff(BitReader& br, const Huff& h) {
  int code = 0;
  for (int l = 1; l <= 16; ++l) {
    code = (code << 1) | br.bit();
    if (h.maxcode[l] >= 0 && code <= h.maxcode[l] && code >= h.mincode[l]) {
      const int idx = h.valptr[l] + code - h.mincode[l];
      return idx >= 0 && idx < 256 ? h.vals[idx] : -1;
    }
    if (br.marker) return -1;
  }
  return -1;
}
// value of a `t`-bit magnitude category (1 <= t <= 15)
static inline int extend(int v, int t) { return v < (1 << (t - 1)) ? v - (1 << t) + 1 : v; }

struct IdctTable {
  float c[8][8];
  IdctTable() { for (int x = 0; x < 8; ++x) for (int u = 0; u < 8; ++u) c[x][u] = (u == 0 ? std::sqrt(0.125f) : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979f / 16.f); }
};
static void idct8x8(const float* in, uint8_t* out, int stride) {
  // separable float IDCT on the exact cosine basis: within +-1 of libjpeg's slow integer IDCT.  The table is a
  // function-local static: initialised once, thread-safe (several decode workers run at the same time).
  static const IdctTable tab;
  const float (*c)[8] = tab.c;
  float tmp[64];
  for (int y = 0; y < 8; ++y)
    for (int x = 0; x < 8; ++x) { float s = 0; for (int u = 0; u < 8; ++u) s += c[x][u] * in[y * 8 + u]; tmp[y * 8 + x] = s; }
  for (int x = 0; x < 8; ++x)
    for (int y = 0; y < 8; ++y) {
      float s = 0; for (int v = 0; v < 8; ++v) s += c[y][v] * tmp[v * 8 + x];
      int o = (int)std::lrintf(s + 128.f);
      out[y * stride + x] = (uint8_t)(o < 0 ? 0 : o > 255 ? 255 : o);
    }
}

// One block of one scan.  Returns false when the entropy-coded data ends or is malformed (the caller keeps what has been
// decoded so far).  `eobrun` carries the end-of-band run of progressive AC scans across blocks.
static bool decode_block(BitReader& br, Comp& c, int16_t* blk, const Huff* dc, const Huff* ac, bool progressive, int Ss, int Se, int Ah, int Al,
                         int& eobrun) {
  if (!progressive) {
    int t = decode_huff(br, dc[c.td]);
    if (t < 0 || t > 11) return false;
    int diff = t ? extend(br.bits(t), t) : 0;
    c.dc_pred += diff;
    blk[0] = (int16_t)c.dc_pred;
    for (int k = 1; k < 64;) {
      int rs = decode_huff(br, ac[c.ta]);
      if (rs < 0) return false;
      int r = rs >> 4, s = rs & 15;
      if (s == 0) { if (r == 15) { k += 16; continue; } break; }
      k += r;
      if (k > 63) return false;
      blk[kZigzag[k]] = (int16_t)extend(br.bits(s), s);
      ++k;
    }
    return true;
  }
  if (Ss == 0) {                                   // DC scan
    if (Ah == 0) {
      int t = decode_huff(br, dc[c.td]);
      if (t < 0 || t > 11) return false;
      int diff = t ? extend(br.bits(t), t) : 0;
      c.dc_pred += diff;
      blk[0] = (int16_t)(c.dc_pred * (1 << Al));
    } else if (br.bit()) {
      blk[0] = (int16_t)(blk[0] | (1 << Al));
    }
    return true;
  }
  const int bit = 1 << Al;
  if (Ah == 0) {                                   // AC scan, first pass of a band
    if (eobrun > 0) { --eobrun; return true; }
    for (int k = Ss; k <= Se;) {
      int rs = decode_huff(br, ac[c.ta]);
      if (rs < 0) return false;
      int r = rs >> 4, s = rs & 15;
      if (s == 0) {
        if (r < 15) { eobrun = (1 << r) - 1; if (r) eobrun += br.bits(r); break; }
        k += 16;
      } else {
        k += r;
        if (k > Se) return false;
        blk[kZigzag[k]] = (int16_t)(extend(br.bits(s), s) * bit);
        ++k;
      }
    }
    return true;
  }
  // AC scan, refinement of a band
  auto refine = [&](int16_t& v) { if (br.bit() && (v & bit) == 0) v = (int16_t)(v + (v > 0 ? bit : -bit)); };
  if (eobrun > 0) {
    --eobrun;
    for (int k = Ss; k <= Se; ++k) { int16_t& v = blk[kZigzag[k]]; if (v != 0) refine(v); }
    return true;
  }
  for (int k = Ss; k <= Se;) {
    int rs = decode_huff(br, ac[c.ta]);
    if (rs < 0) return false;
    int r = rs >> 4, s = rs & 15, val = 0;
    if (s == 0) {
      if (r < 15) { eobrun = (1 << r) - 1; if (r) eobrun += br.bits(r); r = 64; }      // the rest of the band: corrections only
    } else {
      if (s != 1) return false;
      val = br.bit() ? bit : -bit;
    }
    while (k <= Se) {
      int16_t& v = blk[kZigzag[k++]];
      if (v != 0) refine(v);
      else { if (r == 0) { v = (int16_t)val; break; } --r; }
    }
  }
  return true;
}

// Decodes into interleaved RGB. Returns 0, or a negative code: -1 malformed, -2 unsupported (arithmetic coding, lossless,
// hierarchical, 12-bit samples, sampling factors above 4).
static int jpeg_decode(const uint8_t* data, size_t size, std::vector<uint8_t>& rgb, int& W, int& H) {
  if (size < 4 || data[0] != 0xFF || data[1] != 0xD8) return -1;
  uint16_t qt[4][64]; bool qset[4] = {false, false, false, false};
  Huff dc[4], ac[4];
  std::vector<Comp> comps;
  int restart = 0, hmax = 1, vmax = 1, mx = 0, my = 0;
  bool progressive = false, adobe = false; int adobe_transform = -1;
  int scans = 0;
  unsigned seen = 0;
  size_t pos = 2;
  W = H = 0;
  while (pos + 4 <= size) {
    if (data[pos] != 0xFF) { ++pos; continue; }
    uint8_t m = data[pos + 1];
    pos += 2;
    if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01 || m == 0xFF) { if (m == 0xFF) --pos; continue; }
    if (m == 0xD9) break;
    if (pos + 2 > size) break;
    size_t len = ((size_t)data[pos] << 8) | data[pos + 1];
    if (len < 2 || pos + len > size) { if (scans) break; return -1; }
    const uint8_t* seg = data + pos + 2; size_t sl = len - 2;
    if (m == 0xDB) {
      size_t i = 0;
      while (i < sl) {
        int pq = seg[i] >> 4, tq = seg[i] & 15; ++i;
        if (tq > 3 || pq > 1) return -1;
        for (int k = 0; k < 64; ++k) {
          if (i + (pq ? 2 : 1) > sl) return -1;
          qt[tq][kZigzag[k]] = pq ? (uint16_t)((seg[i] << 8) | seg[i + 1]) : seg[i];
          i += pq ? 2 : 1;
        }
        qset[tq] = true;
      }
    } else if (m == 0xC4) {
      size_t i = 0;
      while (i + 17 <= sl) {
        int tc = seg[i] >> 4, th = seg[i] & 15; ++i;
        if (th > 3 || tc > 1) return -1;
        Huff& h = tc ? ac[th] : dc[th];
        int total = 0; h.bits[0] = 0;
        for (int l = 1; l <= 16; ++l) { h.bits[l] = seg[i++]; total += h.bits[l]; }
        if (total > 256 || i + total > sl) return -1;
        memset(h.vals, 0, sizeof h.vals);
        memcpy(h.vals, seg + i, total); i += total;
        build_huff(h);
      }
    } else if (m == 0xC0 || m == 0xC1 || m == 0xC2) {
      if (!comps.empty()) return -1;                           // one frame per file
      if (sl < 6 || seg[0] != 8) return -2;
      progressive = m == 0xC2;
      H = (seg[1] << 8) | seg[2]; W = (seg[3] << 8) | seg[4];
      int nc = seg[5];
      if ((nc != 1 && nc != 3 && nc != 4) || sl < (size_t)(6 + 3 * nc) || W <= 0 || H <= 0) return -2;
      if ((long long)W * H > (1LL << 28)) return -2;
      comps.resize(nc);
      for (int i = 0; i < nc; ++i) {
        comps[i].id = seg[6 + 3 * i]; comps[i].h = seg[7 + 3 * i] >> 4; comps[i].v = seg[7 + 3 * i] & 15; comps[i].tq = seg[8 + 3 * i];
        if (comps[i].h < 1 || comps[i].h > 4 || comps[i].v < 1 || comps[i].v > 4) return -2;
        if (comps[i].tq > 3) return -1;
        hmax = std::max(hmax, comps[i].h); vmax = std::max(vmax, comps[i].v);
      }
      mx = (W + 8 * hmax - 1) / (8 * hmax); my = (H + 8 * vmax - 1) / (8 * vmax);
      for (auto& c : comps) {
        c.bw = mx * c.h; c.bh = my * c.v;
        c.cw = (W * c.h + hmax - 1) / hmax; c.ch = (H * c.v + vmax - 1) / vmax;
        c.coef.assign((size_t)c.bw * c.bh * 64, 0);
      }
    } else if (m >= 0xC3 && m <= 0xCF && m != 0xC4 && m != 0xC8 && m != 0xCC) {
      return -2;                                               // lossless, hierarchical, arithmetic coding
    } else if (m == 0xDD) {
      if (sl < 2) return -1;
      restart = (seg[0] << 8) | seg[1];
    } else if (m == 0xEE) {
      if (sl >= 12 && memcmp(seg, "Adobe", 5) == 0) { adobe = true; adobe_transform = seg[11]; }
    } else if (m == 0xDA) {
      if (comps.empty() || sl < 1) return -1;
      const int ns = seg[0];
      if (ns < 1 || ns > (int)comps.size() || sl < (size_t)(1 + 2 * ns + 3)) return -1;
      Comp* sc[4];
      for (int i = 0; i < ns; ++i) {
        const int cid = seg[1 + 2 * i];
        sc[i] = nullptr;
        for (auto& c : comps) if (c.id == cid) sc[i] = &c;
        if (!sc[i]) return -1;                                 // the scan names a component the frame does not have
        for (int j = 0; j < i; ++j) if (sc[j] == sc[i]) return -1;
        sc[i]->td = seg[2 + 2 * i] >> 4; sc[i]->ta = seg[2 + 2 * i] & 15;
        if (sc[i]->td > 3 || sc[i]->ta > 3) return -1;
      }
      int Ss = seg[1 + 2 * ns], Se = seg[2 + 2 * ns], Ah = seg[3 + 2 * ns] >> 4, Al = seg[3 + 2 * ns] & 15;
      if (!progressive) { Ss = 0; Se = 63; Ah = Al = 0; }
      else if (Ss > Se || Se > 63 || Al > 13 || Ah > 13 || (Ss == 0 && Se != 0) || (Ss > 0 && ns != 1)) return -1;
      for (int i = 0; i < ns; ++i) {
        const bool need_dc = !progressive || Ss == 0, need_ac = !progressive || Ss > 0;
        if ((need_dc && Ah == 0 && !dc[sc[i]->td].set) || (need_ac && !ac[sc[i]->ta].set)) return -1;
        sc[i]->dc_pred = 0;
      }
      BitReader br{data + pos + len, data + size};
      int count = 0, eobrun = 0;
      bool ok = true;
      auto restart_if_due = [&]() {
        if (!restart || count != restart) return;
        br.reset();
        while (br.p + 1 < br.end && !(br.p[0] == 0xFF && br.p[1] >= 0xD0 && br.p[1] <= 0xD7)) ++br.p;
        if (br.p + 1 < br.end) br.p += 2;
        for (int i = 0; i < ns; ++i) sc[i]->dc_pred = 0;
        eobrun = 0; count = 0;
      };
      if (ns == 1) {
        // a scan of one component walks that component's own blocks (those that hold image samples), row by row
        Comp& c = *sc[0];
        const int nbx = (c.cw + 7) / 8, nby = (c.ch + 7) / 8;
        for (int by = 0; by < nby && ok; ++by)
          for (int bx = 0; bx < nbx && ok; ++bx) {
            restart_if_due();
            ok = decode_block(br, c, &c.coef[((size_t)by * c.bw + bx) * 64], dc, ac, progressive, Ss, Se, Ah, Al, eobrun);
            ++count;
          }
      } else {
        for (int row = 0; row < my && ok; ++row)
          for (int col = 0; col < mx && ok; ++col) {
            restart_if_due();
            for (int i = 0; i < ns && ok; ++i) {
              Comp& c = *sc[i];
              for (int by = 0; by < c.v && ok; ++by)
                for (int bx = 0; bx < c.h && ok; ++bx)
                  ok = decode_block(br, c, &c.coef[((size_t)(row * c.v + by) * c.bw + (col * c.h + bx)) * 64], dc, ac, progressive, Ss, Se, Ah, Al, eobrun);
            }
            ++count;
          }
      }
      ++scans;
      // carry on behind the entropy-coded data: the next marker that is neither a stuffed byte nor a restart marker
      size_t q = (size_t)(br.p - data);
      while (q + 1 < size && !(data[q] == 0xFF && data[q + 1] != 0x00 && !(data[q + 1] >= 0xD0 && data[q + 1] <= 0xD7) && data[q + 1] != 0xFF)) ++q;
      pos = q;
      if (!progressive) {                                      // a sequential frame is complete once every component has had its scan
        for (int i = 0; i < ns; ++i) seen |= 1u << (int)(sc[i] - comps.data());
        if (seen == (1u << comps.size()) - 1u) break;
      }
      continue;
    }
    pos += len;
  }
  if (comps.empty() || scans == 0) return -1;
  for (auto& c : comps) if (!qset[c.tq]) return -1;
  // ---- coefficients -> samples -----------------------------------------------------------------------------------------
  {
    float blk[64];
    for (auto& c : comps) {
      c.pw = c.bw * 8; c.ph = c.bh * 8;
      c.plane.assign((size_t)c.pw * c.ph, 128);
      const int nbx = (c.cw + 7) / 8, nby = (c.ch + 7) / 8;
      for (int by = 0; by < nby; ++by)
        for (int bx = 0; bx < nbx; ++bx) {
          const int16_t* q = &c.coef[((size_t)by * c.bw + bx) * 64];
          for (int k = 0; k < 64; ++k) blk[k] = (float)((int)q[k] * (int)qt[c.tq][k]);
          idct8x8(blk, c.plane.data() + (size_t)(by * 8) * c.pw + bx * 8, c.pw);
        }
      std::vector<int16_t>().swap(c.coef);
    }
  }
  // chroma up-sampling (libjpeg's "fancy" triangle filter for 2:1 factors, replication otherwise) + colour conversion
  {
    std::vector<std::vector<uint8_t>> full(comps.size());
    for (size_t ci = 0; ci < comps.size(); ++ci) {
      Comp& c = comps[ci];
      const int cw = c.cw, chh = c.ch;
      std::vector<uint8_t>& out = full[ci];
      out.resize((size_t)W * H);
      const bool h2 = c.h * 2 == hmax, v2 = c.v * 2 == vmax, h1 = c.h == hmax, v1 = c.v == vmax;
      if (h1 && v1) {
        for (int y = 0; y < H; ++y) memcpy(&out[(size_t)y * W], &c.plane[(size_t)y * c.pw], (size_t)W);
      } else if (h2 && (v1 || v2)) {
        std::vector<int> colsum((size_t)cw);
        for (int y = 0; y < H; ++y) {
          // vertical: nearer row weight 3, farther row weight 1 (v2), or the row itself times 4 (v1)
          int yn = v2 ? y / 2 : y;
          int yf = v2 ? ((y & 1) ? std::min(yn + 1, chh - 1) : std::max(yn - 1, 0)) : yn;
          const uint8_t* rn = &c.plane[(size_t)yn * c.pw]; const uint8_t* rf = &c.plane[(size_t)yf * c.pw];
          for (int x = 0; x < cw; ++x) colsum[x] = v2 ? 3 * rn[x] + rf[x] : rn[x];
          uint8_t* o = &out[(size_t)y * W];
          for (int x = 0; x < W; ++x) {
            int i = x / 2, t = colsum[i];
            int v;
            if (v2) {
              if (cw == 1) v = (t * 4 + 8) >> 4;
              else if (!(x & 1)) v = i == 0 ? (t * 4 + 8) >> 4 : (t * 3 + colsum[i - 1] + 8) >> 4;
              else v = i == cw - 1 ? (t * 4 + 7) >> 4 : (t * 3 + colsum[i + 1] + 7) >> 4;
            } else {
              if (cw == 1) v = t;
              else if (!(x & 1)) v = i == 0 ? t : (t * 3 + colsum[i - 1] + 1) >> 2;
              else v = i == cw - 1 ? t : (t * 3 + colsum[i + 1] + 2) >> 2;
            }
            o[x] = (uint8_t)v;
          }
        }
      } else {
        for (int y = 0; y < H; ++y)
          for (int x = 0; x < W; ++x) {
            const int sy = std::min(chh - 1, y * c.v / vmax), sx = std::min(cw - 1, x * c.h / hmax);
            out[(size_t)y * W + x] = c.plane[(size_t)sy * c.pw + sx];
          }
      }
    }
    const size_t nc = comps.size();
    // three components are YCbCr unless an Adobe marker says "no transform" (or the component ids spell R, G, B);
    // four are CMYK, or YCCK when the Adobe transform code is 2
    const bool ycc3 = nc == 3 && !(adobe && adobe_transform == 0) && !(comps[0].id == 'R' && comps[1].id == 'G' && comps[2].id == 'B');
    const bool ycck = nc == 4 && adobe && adobe_transform == 2;
    auto ycc_to_rgb = [](int Y, int cb, int cr, int& r, int& g, int& b) {
      // libjpeg's fixed-point YCbCr -> RGB (16-bit fractions, rounded)
      cb -= 128; cr -= 128;
      r = Y + ((91881 * cr + 32768) >> 16);
      g = Y + ((-22554 * cb - 46802 * cr + 32768) >> 16);
      b = Y + ((116130 * cb + 32768) >> 16);
      r = std::min(255, std::max(0, r)); g = std::min(255, std::max(0, g)); b = std::min(255, std::max(0, b));
    };
    rgb.resize((size_t)W * H * 3);
    for (size_t i = 0; i < (size_t)W * H; ++i) {
      uint8_t* o = &rgb[i * 3];
      if (nc == 1) { o[0] = o[1] = o[2] = full[0][i]; continue; }
      if (nc == 3) {
        int r = full[0][i], g = full[1][i], b = full[2][i];
        if (ycc3) ycc_to_rgb(full[0][i], full[1][i], full[2][i], r, g, b);
        o[0] = (uint8_t)r; o[1] = (uint8_t)g; o[2] = (uint8_t)b;
        continue;
      }
      // four components: bring them to C, M, Y, K as libjpeg hands them out, then the reference's conversion
      // (image/image.c:119-139: Adobe files store inverted inks, r = k * c / 255; otherwise r = (255 - k)(255 - c) / 255)
      int c = full[0][i], mm = full[1][i], y = full[2][i];
      const int k = full[3][i];
      if (ycck) { int r, g, b; ycc_to_rgb(c, mm, y, r, g, b); c = 255 - r; mm = 255 - g; y = 255 - b; }
      if (adobe) { o[0] = (uint8_t)(k * c / 255); o[1] = (uint8_t)(k * mm / 255); o[2] = (uint8_t)(k * y / 255); }
      else { o[0] = (uint8_t)((255 - k) * (255 - c) / 255); o[1] = (uint8_t)((255 - k) * (255 - mm) / 255); o[2] = (uint8_t)((255 - k) * (255 - y) / 255); }
    }
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Image operations (float, interleaved HWC)
// ---------------------------------------------------------------------------------------------------------------------
struct Rng {           // splitmix64: one independent stream per (seed, record)
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed) {}
  uint64_t next() { uint64_t z = (s += 0x9E3779B97F4A7C15ull); z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; return z ^ (z >> 31); }
  float uniform(float lo, float hi) { return lo + (hi - lo) * (float)((next() >> 40) * (1.0 / 16777216.0)); }
};
struct Box { float xmin, ymin, xmax, ymax; };   // normalised [0,1]

// Random crop with the distribution of the reference's sampler (image/image.c:826-975, itself a restatement of
// tf.image.sample_distorted_bounding_box): per attempt an aspect ratio uniform in [ar_lo, ar_hi]; the HEIGHT uniform over
// the integers between the heights that the smallest and the largest allowed area imply for that ratio (the largest
// lowered until the rounded width fits the image); width = round(height * ratio); one more row if rounding took the area
// below the minimum; the position uniform over the placements that fit; accepted when some labelled box (in whole
// pixels) covers at least `min_cover` of the CROP's area.  After `attempts` failures the whole image is used.
struct PixelRect { int x0, y0, x1, y1; };
static PixelRect sample_distorted_box(Rng& rng, const std::vector<Box>& boxes, int W, int H, float min_cover = 0.1f, float ar_lo = 0.75f, float ar_hi = 1.33f,
                                      float area_lo = 0.05f, float area_hi = 1.0f, int attempts = 100) {
  std::vector<PixelRect> rects;
  for (const Box& b : boxes) rects.push_back({(int)(b.xmin * W), (int)(b.ymin * H), (int)(b.xmax * W), (int)(b.ymax * H)});
  if (rects.empty()) rects.push_back({0, 0, W, H});
  auto uniform_int = [&](int n) { return n <= 0 ? 0 : (int)(rng.next() % (uint64_t)(n + 1)); };      // closed range [0, n]
  const float min_area = area_lo * W * H, max_area = area_hi * W * H;
  for (int a = 0; a < attempts; ++a) {
    const float ratio = rng.uniform(ar_lo, ar_hi);
    int hmin = (int)std::lrintf(std::sqrt(min_area / ratio)), hmax = (int)std::lrintf(std::sqrt(max_area / ratio));
    if (std::lrintf(hmax * ratio) > W) hmax = (int)((W + 0.5 - 1e-7) / ratio);
    hmax = std::min(hmax, H);
    hmin = std::min(hmin, hmax);
    int h = hmin + uniform_int(hmax - hmin);
    int w = (int)std::lrintf(h * ratio);
    if (w > W) continue;
    if ((float)(h * w) < min_area) { h += 1; w = (int)std::lrintf(h * ratio); }
    const float area = (float)(h * w);
    if (area < min_area || area > max_area || w <= 0 || w > W || h <= 0 || h > H) continue;
    const int y = uniform_int(H - h), x = uniform_int(W - w);
    const PixelRect c{x, y, x + w, y + h};
    for (const PixelRect& r : rects) {
      if (r.x1 - r.x0 < 1 || r.y1 - r.y0 < 1) continue;
      const int ix = std::max(0, std::min(c.x1, r.x1) - std::max(c.x0, r.x0)), iy = std::max(0, std::min(c.y1, r.y1) - std::max(c.y0, r.y0));
      if ((float)ix * (float)iy / area >= min_cover) return c;
    }
  }
  return {0, 0, W, H};
}

// bilinear resize of the crop [x0,x0+cw) x [y0,y0+ch) of an interleaved uint8 RGB image into S x S planar floats,
// with optional horizontal flip and the x/127.5 - 1 scaling (half-pixel centres are NOT used, as in TF1's resize_bilinear)
static void crop_resize_to_chw(const uint8_t* rgb, int W, int H, int x0, int y0, int cw, int ch, bool flip, int S, float* out) {
  const float sx = (float)cw / S, sy = (float)ch / S;
  for (int oy = 0; oy < S; ++oy) {
    float fy = oy * sy; int iy = (int)fy; float wy = fy - iy; int iy1 = std::min(iy + 1, ch - 1);
    for (int ox = 0; ox < S; ++ox) {
      int sxp = flip ? (S - 1 - ox) : ox;
      float fx = sxp * sx; int ix = (int)fx; float wx = fx - ix; int ix1 = std::min(ix + 1, cw - 1);
      const uint8_t* p00 = rgb + ((size_t)(y0 + iy) * W + x0 + ix) * 3; const uint8_t* p01 = rgb + ((size_t)(y0 + iy) * W + x0 + ix1) * 3;
      const uint8_t* p10 = rgb + ((size_t)(y0 + iy1) * W + x0 + ix) * 3; const uint8_t* p11 = rgb + ((size_t)(y0 + iy1) * W + x0 + ix1) * 3;
      for (int c = 0; c < 3; ++c) {
        float top = p00[c] + (p01[c] - p00[c]) * wx, bot = p10[c] + (p11[c] - p10[c]) * wx;
        out[((size_t)c * S + oy) * S + ox] = (top + (bot - top) * wy) * (1.f / 127.5f) - 1.f;
      }
    }
  }
}

struct Record { int label; std::vector<Box> boxes; int height, width; const uint8_t* jpeg; size_t jpeg_bytes; };

// Which part of a decoded W x H image becomes the example: the crop window and whether it is mirrored.  The same plan
// drives the CPU path below and the CUDA kernel (csrc/kernels/image.cu), so the two produce identical examples.
struct CropPlan { int x0, y0, cw, ch, flip; };
static CropPlan plan_crop(int W, int H, const std::vector<Box>& boxes, bool training, uint64_t seed) {
  if (training) {
    Rng rng(seed);
    const PixelRect c = sample_distorted_box(rng, boxes, W, H);
    const int flip = (int)(rng.next() & 1);
    return {c.x0, c.y0, std::max(1, c.x1 - c.x0), std::max(1, c.y1 - c.y0), flip};
  }
  // shorter side -> 1.145 * S, then centre crop: equivalent to resizing a centred square crop of side min(W,H)/1.145
  const float side = std::min(W, H) / 1.145f;
  const int cs = std::max(1, (int)std::lrintf(side));
  return {(W - cs) / 2, (H - cs) / 2, cs, cs, 0};
}

// Process one record into out[3*S*S]; returns 0 or the decoder's error code (the output is then a grey image).
static int process_record(const Record& r, bool training, int S, uint64_t seed, float* out) {
  std::vector<uint8_t> rgb; int W = 0, H = 0;
  int e = jpeg_decode(r.jpeg, r.jpeg_bytes, rgb, W, H);
  if (e != 0) { for (size_t i = 0; i < (size_t)3 * S * S; ++i) out[i] = 0.f; return e; }
  const CropPlan p = plan_crop(W, H, r.boxes, training, seed);
  crop_resize_to_chw(rgb.data(), W, H, p.x0, p.y0, p.cw, p.ch, p.flip != 0, S, out);
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Record file
// ---------------------------------------------------------------------------------------------------------------------
struct RecordFile {
  std::vector<uint8_t> bytes;
  std::vector<size_t> offsets;       // start of each record (at its length field)
  bool load(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END); long n = ftell(f); fseek(f, 0, SEEK_SET);
    bytes.resize((size_t)n);
    bool ok = fread(bytes.data(), 1, (size_t)n, f) == (size_t)n;
    fclose(f);
    if (!ok || n < 4) return false;
    int32_t count; memcpy(&count, bytes.data(), 4);
    size_t pos = 4;
    for (int i = 0; i < count; ++i) {
      if (pos + 4 > bytes.size()) return false;
      int32_t len; memcpy(&len, &bytes[pos], 4);
      if (len < 16 || pos + 4 + (size_t)len > bytes.size()) return false;
      offsets.push_back(pos);
      pos += 4 + (size_t)len;
    }
    return true;
  }
  bool get(size_t i, Record& r) const {
    size_t pos = offsets[i];
    int32_t len, label, nb; memcpy(&len, &bytes[pos], 4); memcpy(&label, &bytes[pos + 4], 4); memcpy(&nb, &bytes[pos + 8], 4);
    if (nb < 0 || (size_t)(12 + 16 * nb + 8) > (size_t)len + 4) return false;
    r.label = label; r.boxes.resize(nb);
    const uint8_t* p = &bytes[pos + 12];
    for (int k = 0; k < nb; ++k) { memcpy(&r.boxes[k].xmin, p + 4 * k, 4); memcpy(&r.boxes[k].ymin, p + 4 * (nb + k), 4); memcpy(&r.boxes[k].xmax, p + 4 * (2 * nb + k), 4); memcpy(&r.boxes[k].ymax, p + 4 * (3 * nb + k), 4); }
    p += 16 * nb;
    memcpy(&r.height, p, 4); memcpy(&r.width, p + 4, 4);
    r.jpeg = p + 8; r.jpeg_bytes = (size_t)len - (8 + 16 * nb + 8);
    return true;
  }
};

// ---------------------------------------------------------------------------------------------------------------------
// Double-buffered record data set
// ---------------------------------------------------------------------------------------------------------------------
struct RecordDataset {
  std::vector<RecordFile> files;
  std::vector<std::pair<int, int>> index;      // (file, record) of every example, shuffled per epoch
  int batch, NB, S, workers; bool training; uint64_t seed;
  size_t img_floats, batch_ex_bytes, batch_lab_bytes;
  char* ex[2] = {nullptr, nullptr}; char* lab[2] = {nullptr, nullptr};
  std::atomic<int> ready[2];                   // half filled and not yet handed out completely
  std::atomic<long long> inflight[2];          // tasks reading from this half (count-down latch)
  std::atomic<long long> fill_group{0};        // next group of NB batches to decode
  std::atomic<bool> running{true};
  std::atomic<long long> decode_failures{0}, images{0};
  std::thread filler;
  long long epoch_len() const { return (long long)index.size() / batch; }

  void shuffle(uint64_t epoch) {
    Rng r(seed ^ (0x5851F42D4C957F2Dull * (epoch + 1)));
    for (size_t i = index.size(); i > 1; --i) std::swap(index[i - 1], index[r.next() % i]);
  }
  void fill_half(int half, long long group) {
    const long long first = group * NB * batch;
    const long long total = (long long)NB * batch;
    std::atomic<long long> next{0};
    auto work = [&]() {
      for (;;) {
        long long i = next.fetch_add(1);
        if (i >= total) return;
        long long g = (first + i) % (long long)index.size();
        auto fr = index[(size_t)g];
        Record rec;
        long long b = i / batch, j = i % batch;
        float* dst = (float*)(ex[half] + (size_t)b * batch_ex_bytes) + (size_t)j * img_floats;
        int32_t* ldst = (int32_t*)(lab[half] + (size_t)b * batch_lab_bytes) + j;
        if (!files[fr.first].get((size_t)fr.second, rec)) { decode_failures.fetch_add(1); *ldst = 0; continue; }
        if (process_record(rec, training, S, seed + 0x9E3779B97F4A7C15ull * (uint64_t)(first + i + 1), dst) != 0) decode_failures.fetch_add(1);
        *ldst = rec.label;
        images.fetch_add(1);
      }
    };
    std::vector<std::thread> ts;
    for (int w = 1; w < workers; ++w) ts.emplace_back(work);
    work();
    for (auto& t : ts) t.join();
  }
  void filler_loop() {
    unsigned spins = 0;
    while (running.load()) {
      long long g = fill_group.load();
      int half = (int)(g & 1);
      if (ready[half].load() == 0 && inflight[half].load() == 0) {
        if (training && NB * batch > 0 && (g * NB) % std::max<long long>(1, epoch_len()) < NB) shuffle((uint64_t)((g * NB) / std::max<long long>(1, epoch_len())));
        fill_half(half, g);
        ready[half].store(1, std::memory_order_release);
        fill_group.store(g + 1);
        spins = 0;
      } else cpu_relax(++spins);
    }
  }
  // batch b (global, monotonically increasing): returns the half it lives in, or -1 on timeout
  int take(long long b, const void** e, const void** l, double timeout_s) {
    long long g = b / NB; int half = (int)(g & 1);
    auto t0 = Clock::now(); unsigned spins = 0;
    while (!(ready[half].load(std::memory_order_acquire) == 1 && fill_group.load() > g)) {
      cpu_relax(++spins);
      if (seconds_since(t0) > timeout_s) return -1;
    }
    inflight[half].fetch_add(1);
    long long i = b % NB;
    *e = ex[half] + (size_t)i * batch_ex_bytes; *l = lab[half] + (size_t)i * batch_lab_bytes;
    if (i == NB - 1) ready[half].store(0, std::memory_order_release);     // last batch of the half handed out: refill once the latch drops
    return half;
  }
  void release(int half) { inflight[half].fetch_sub(1); }
};

}  // namespace xb

using namespace xb;

// ---- C ABI --------------------------------------------------------------------------------------------------------------
RT_API int rec_jpeg_decode(const void* data, long long size, unsigned char* rgb_out, long long capacity, int* w, int* h) {
  std::vector<uint8_t> rgb; int W, H;
  int e = jpeg_decode((const uint8_t*)data, (size_t)size, rgb, W, H);
  *w = W; *h = H;
  if (e != 0) return e;
  if ((long long)rgb.size() > capacity) return -3;
  memcpy(rgb_out, rgb.data(), rgb.size());
  return 0;
}
RT_API int rec_process(const void* jpeg, long long size, const float* boxes_xyxy, int nboxes, int training, int S, unsigned long long seed, float* out) {
  Record r; r.label = 0; r.jpeg = (const uint8_t*)jpeg; r.jpeg_bytes = (size_t)size; r.height = r.width = 0;
  for (int i = 0; i < nboxes; ++i) r.boxes.push_back({boxes_xyxy[4 * i], boxes_xyxy[4 * i + 1], boxes_xyxy[4 * i + 2], boxes_xyxy[4 * i + 3]});
  return process_record(r, training != 0, S, seed, out);
}
// writer
struct RecWriter { FILE* f; int32_t count; };
// Crop plan of one decoded image (x0, y0, width, height, flip) for the given boxes / phase / seed: what rec_process uses.
RT_API void rec_plan(int W, int H, const float* boxes_xyxy, int nboxes, int training, unsigned long long seed, int* plan5) {
  std::vector<Box> boxes((size_t)(nboxes > 0 ? nboxes : 0));
  for (int k = 0; k < nboxes; ++k) boxes[k] = {boxes_xyxy[4 * k], boxes_xyxy[4 * k + 1], boxes_xyxy[4 * k + 2], boxes_xyxy[4 * k + 3]};
  const CropPlan p = plan_crop(W, H, boxes, training != 0, seed);
  plan5[0] = p.x0; plan5[1] = p.y0; plan5[2] = p.cw; plan5[3] = p.ch; plan5[4] = p.flip;
}

RT_API void* rec_writer_open(const char* path) {
  FILE* f = fopen(path, "wb");
  if (!f) return nullptr;
  int32_t zero = 0; fwrite(&zero, 4, 1, f);
  return new RecWriter{f, 0};
}
RT_API int rec_writer_append(void* wp, const void* jpeg, long long size, int label, const float* boxes_xyxy, int nboxes, int height, int width) {
  RecWriter* w = (RecWriter*)wp;
  int32_t len = (int32_t)(8 + 16 * nboxes + 8 + size), lab = label, nb = nboxes, h = height, wd = width;
  fwrite(&len, 4, 1, w->f); fwrite(&lab, 4, 1, w->f); fwrite(&nb, 4, 1, w->f);
  for (int c = 0; c < 4; ++c) for (int i = 0; i < nboxes; ++i) fwrite(&boxes_xyxy[4 * i + c], 4, 1, w->f);
  fwrite(&h, 4, 1, w->f); fwrite(&wd, 4, 1, w->f);
  fwrite(jpeg, 1, (size_t)size, w->f);
  w->count++;
  return 0;
}
RT_API int rec_writer_close(void* wp) {
  RecWriter* w = (RecWriter*)wp;
  fseek(w->f, 0, SEEK_SET); fwrite(&w->count, 4, 1, w->f);
  int c = w->count; fclose(w->f); delete w; return c;
}
// data set
RT_API void* rec_dataset_open(const char* const* paths, int npaths, int batch, int batches_per_half, int image_size, int workers, int training,
                              unsigned long long seed) {
  RecordDataset* d = new RecordDataset();
  d->files.resize(npaths);
  for (int i = 0; i < npaths; ++i) {
    if (!d->files[i].load(paths[i])) { delete d; return nullptr; }
    for (size_t r = 0; r < d->files[i].offsets.size(); ++r) d->index.push_back({i, (int)r});
  }
  if (d->index.empty() || batch < 1 || batches_per_half < 1) { delete d; return nullptr; }
  d->batch = batch; d->NB = batches_per_half; d->S = image_size; d->workers = workers < 1 ? 1 : workers; d->training = training != 0; d->seed = seed;
  d->img_floats = (size_t)3 * image_size * image_size;
  size_t page = (size_t)sysconf(_SC_PAGESIZE);
  d->batch_ex_bytes = ((size_t)batch * d->img_floats * 4 + page - 1) / page * page;
  d->batch_lab_bytes = ((size_t)batch * 4 + page - 1) / page * page;
  for (int h = 0; h < 2; ++h) {
    if (posix_memalign((void**)&d->ex[h], page, d->batch_ex_bytes * d->NB) || posix_memalign((void**)&d->lab[h], page, d->batch_lab_bytes * d->NB)) { delete d; return nullptr; }
    memset(d->lab[h], 0, d->batch_lab_bytes * d->NB);
    d->ready[h].store(0); d->inflight[h].store(0);
  }
  d->filler = std::thread([d] { d->filler_loop(); });
  return d;
}
RT_API void* rec_dataset_buffer(void* dp, int half, int which, long long* bytes) {
  RecordDataset* d = (RecordDataset*)dp;
  *bytes = (long long)((which == 0 ? d->batch_ex_bytes : d->batch_lab_bytes) * d->NB);
  return which == 0 ? d->ex[half] : d->lab[half];
}
RT_API int rec_dataset_take(void* d, long long b, const void** e, const void** l, double timeout_s) { return ((RecordDataset*)d)->take(b, e, l, timeout_s); }
RT_API void rec_dataset_release(void* d, int half) { ((RecordDataset*)d)->release(half); }
RT_API long long rec_dataset_examples(void* d) { return (long long)((RecordDataset*)d)->index.size(); }
RT_API long long rec_dataset_failures(void* d) { return ((RecordDataset*)d)->decode_failures.load(); }
RT_API long long rec_dataset_images(void* d) { return ((RecordDataset*)d)->images.load(); }
RT_API void rec_dataset_close(void* dp) {
  RecordDataset* d = (RecordDataset*)dp;
  d->running.store(false);
  if (d->filler.joinable()) d->filler.join();
  for (int h = 0; h < 2; ++h) { free(d->ex[h]); free(d->lab[h]); }
  delete d;
}
// adapters for the host runtime's data-source hooks
struct RecSource { void* ds; long long stride, offset; double timeout_s; };
RT_API void* rec_source_create(void* ds, long long stride, long long offset, double timeout_s) { return new RecSource{ds, stride, offset, timeout_s}; }
RT_API void rec_source_free(void* s) { delete (RecSource*)s; }
RT_API int rec_source_take(void* sp, unsigned long long task, int, const void** e, const void** l) {
  RecSource* s = (RecSource*)sp;
  return ((RecordDataset*)s->ds)->take((long long)task * s->stride + s->offset, e, l, s->timeout_s);
}
RT_API void rec_source_release(void* sp, int half) { ((RecordDataset*)((RecSource*)sp)->ds)->release(half); }
