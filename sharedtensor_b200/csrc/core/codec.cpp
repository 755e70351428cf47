// Host implementation of the sign-bit codec; see codec.hpp for the formats and the state model.
// Compiled with -ffp-contract=off so that the fp32 sums match the CUDA kernels, which use
// explicit round-to-nearest multiplies and adds.
#include "codec.hpp"

#include <cmath>
#include <vector>

namespace st {

size_t sign_bytes(size_t n) { return (n + 7) / 8; }
size_t block_words(size_t n) { return (n + 31) / 32; }
size_t block_scales(size_t n, int block) { return (n + size_t(block) - 1) / size_t(block); }

static float pow2_floor(float s) {
  if (!(s > 0.0f) || std::isinf(s)) return 0.0f;
  int e;
  std::frexp(double(s), &e);  // s = m * 2^e, m in [0.5, 1)
  return float(std::ldexp(1.0, e - 1));
}

float ref_scale_of(const float* r, size_t n) {
  float acc = 0.0f;
  for (size_t i = 0; i < n; i++) acc += r[i] * r[i];
  float mean = acc / float(n);
  float rms = float(std::sqrt(double(mean)));
  return pow2_floor(rms);
}

float encode_residual_ref(float* r, size_t n, uint8_t* bits) {
  float scale = ref_scale_of(r, n);
  std::memset(bits, 0, sign_bytes(n));
  for (size_t i = 0; i < n; i++) {
    if (r[i] > 0.0f) {
      r[i] -= scale;
    } else {
      bits[i >> 3] |= uint8_t(1u << (i & 7));
      r[i] += scale;
    }
  }
  return scale;
}

float encode_tensor(const float* v, float* k, size_t n, uint8_t* bits, float min_scale) {
  float acc = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float x = v[i] - k[i];
    acc += x * x;
  }
  float mean = acc / float(n);
  float scale = pow2_floor(float(std::sqrt(double(mean))));
  if (scale < min_scale) scale = 0.0f;
  std::memset(bits, 0, sign_bytes(n));
  if (scale == 0.0f) {
    // A scale-0 frame moves nothing whatever its bits say; keep the reference's convention that
    // non-positive residuals carry bit 1 so captures of idle links look alike.
    for (size_t i = 0; i < n; i++)
      if (!(v[i] - k[i] > 0.0f)) bits[i >> 3] |= uint8_t(1u << (i & 7));
    return 0.0f;
  }
  for (size_t i = 0; i < n; i++) {
    float x = v[i] - k[i];
    if (x > 0.0f) {
      k[i] += scale;
    } else {
      bits[i >> 3] |= uint8_t(1u << (i & 7));
      k[i] -= scale;
    }
  }
  return scale;
}

void decode_tensor_add(const uint8_t* bits, float scale, size_t n, float* dst, float* dst2) {
  if (scale == 0.0f) return;
  const float step[2] = {scale, -scale};
  if (dst2) {
    for (size_t i = 0; i < n; i++) {
      float f = step[(bits[i >> 3] >> (i & 7)) & 1];
      dst[i] += f;
      dst2[i] += f;
    }
  } else {
    for (size_t i = 0; i < n; i++) dst[i] += step[(bits[i >> 3] >> (i & 7)) & 1];
  }
}

float group32_sumsq(const float* x) {
  float p[8];
  for (int q = 0; q < 8; q++) {
    const float* a = x + 4 * q;
    p[q] = (a[0] * a[0] + a[1] * a[1]) + (a[2] * a[2] + a[3] * a[3]);
  }
  // butterfly order of a xor-shuffle reduction over 8 lanes: offsets 1, 2, 4
  float l1[4] = {p[0] + p[1], p[2] + p[3], p[4] + p[5], p[6] + p[7]};
  float l2[2] = {l1[0] + l1[1], l1[2] + l1[3]};
  return l2[0] + l2[1];
}

static float pairwise_tree(const float* s, int m) {
  // m is a power of two <= 128; adjacent pairs, level by level
  float buf[128];
  for (int i = 0; i < m; i++) buf[i] = s[i];
  for (int w = m; w > 1; w >>= 1)
    for (int i = 0; i < w / 2; i++) buf[i] = buf[2 * i] + buf[2 * i + 1];
  return buf[0];
}

static int ilog2(int b) {
  int l = 0;
  while ((1 << l) < b) l++;
  return l;
}

// Decides the exponent code of one block from its residual energy and the largest magnitude among its
// values.  The relative cut-off is tied to the largest element, not to the RMS: a step of at least
// 2^(emax - rel_bits) with rel_bits <= 22 is a whole number of ulps of every element of the block, so
// stepping the mirror is exact and the stream cannot get stuck re-sending a step that rounds away.
static inline int block_code(float sx, uint32_t vmax_bits, int log2_block, const BlockGate& gate) {
  if ((f32_bits(sx) >> 23) == 0) return kSilent;  // zero or denormal energy
  int kx = rms_exponent(sx, log2_block);
  if (kx < gate.min_exp) return kSilent;
  if ((vmax_bits >> 23) != 0) {
    int emax = int(vmax_bits >> 23) - 127;
    if (kx < emax - gate.rel_bits) return kSilent;
  }
  if (kx < kMinExp) return kSilent;
  if (kx > kMaxExp) kx = kMaxExp;
  return kx + 127;
}

double encode_block(const float* v, float* k, size_t n, int block, const BlockGate& gate,
                    uint32_t* words, uint8_t* scales) {
  const int m = block / 32;
  const int lb = ilog2(block);
  const size_t nb = block_scales(n, block);
  double total = 0.0;
  std::vector<float> x(static_cast<size_t>(block), 0.0f), vv(static_cast<size_t>(block), 0.0f);
  float sx32[128];
  for (size_t b = 0; b < nb; b++) {
    size_t base = b * size_t(block);
    for (int j = 0; j < block; j++) {
      size_t i = base + size_t(j);
      if (i < n) {
        vv[j] = v[i];
        x[j] = v[i] - k[i];
      } else {
        vv[j] = 0.0f;
        x[j] = 0.0f;
      }
    }
    for (int g = 0; g < m; g++) sx32[g] = group32_sumsq(&x[size_t(g) * 32]);
    float sx = pairwise_tree(sx32, m);
    uint32_t vmax = 0;
    for (int j = 0; j < block; j++) {
      uint32_t a = f32_bits(vv[j]) & 0x7fffffffu;
      if (a > vmax) vmax = a;
    }
    total += double(sx);
    // The last block may be partly padding: its RMS is taken over the next power of two that
    // holds its valid elements, so that the zeros do not dilute the scale.
    int lb_eff = lb;
    if (base + size_t(block) > n) lb_eff = ilog2(int(n - base));
    int code = block_code(sx, vmax, lb_eff, gate);
    scales[b] = uint8_t(code);
    float scale = code ? exp2i(code - 127) : 0.0f;
    for (int g = 0; g < m; g++) {
      size_t wbase = base + size_t(g) * 32;
      if (wbase >= n) break;
      uint32_t w = 0;
      for (int j = 0; j < 32; j++) {
        size_t i = wbase + size_t(j);
        if (i >= n) break;
        bool neg = !(x[size_t(g) * 32 + j] > 0.0f);
        if (neg) w |= 1u << j;
        if (code) k[i] += neg ? -scale : scale;
      }
      words[wbase / 32] = w;
    }
  }
  return total;
}

void decode_block_add(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* dst,
                      float* dst2) {
  const size_t nb = block_scales(n, block);
  for (size_t b = 0; b < nb; b++) {
    int code = scales[b];
    if (!code) continue;
    float scale = exp2i(code - 127);
    size_t base = b * size_t(block);
    size_t end = base + size_t(block) < n ? base + size_t(block) : n;
    for (size_t i = base; i < end; i++) {
      float f = ((words[i >> 5] >> (i & 31)) & 1u) ? -scale : scale;
      dst[i] += f;
      if (dst2) dst2[i] += f;
    }
  }
}

void segment_sumsq(const float* x, const int64_t* offsets, int n_seg, double* out) {
  for (int s = 0; s < n_seg; s++) {
    double acc = 0.0;
    for (int64_t i = offsets[s]; i < offsets[s + 1]; i++) acc += double(x[i]) * double(x[i]);
    out[s] = acc;
  }
}

}  // namespace st
