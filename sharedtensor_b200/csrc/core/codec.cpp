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

float encode_tensor(const float* v, float* k, size_t n, uint8_t* bits, float min_scale, int rule) {
  float scale;
  if (rule == 0) {  // the reference's rule: power-of-two floor of the RMS
    float acc = 0.0f;
    for (size_t i = 0; i < n; i++) {
      float x = v[i] - k[i];
      acc += x * x;
    }
    float mean = acc / float(n);
    scale = pow2_floor(float(std::sqrt(double(mean))));
  } else {          // bisection: power-of-two floor of two thirds of the largest residual
    float xmax = 0.0f;
    for (size_t i = 0; i < n; i++) {
      float ax = std::fabs(v[i] - k[i]);
      if (ax > xmax) xmax = ax;
    }
    scale = pow2_floor(xmax * 0.6666667f);
  }
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

// Decides the exponent code of one block from its largest residual magnitude and the largest magnitude among
// its values.
//
// Step rule: 2^floor(log2(2/3 * max|x|)), i.e. between a third and two thirds of the largest residual.  Every
// element moves by that step towards zero or past it, so after the pass no residual exceeds max(step, max - step)
// <= 2/3 max, and from the second pass on the bound halves with every pass (bisection).  The reference takes
// the power-of-two floor of the RMS instead (src/sharedtensor.c:156-159), which never overshoots but removes
// only ~16 % of the error per frame and leaves outliers for hundreds of frames.
//
// Cut-off: a step below 2^(emax - rel_bits), emax the exponent of the block's largest |value|, is not sent.
// With rel_bits <= 22 every step is a whole number of ulps of every element of the block, so stepping the
// mirror is exact and the stream cannot get stuck re-sending a step that rounds away.
int block_code(float xmax, uint32_t vmax_bits, const BlockGate& gate) {
  float scaled = xmax * 0.6666667f;
  if ((f32_bits(scaled) >> 23) == 0) return kSilent;  // zero or denormal
  int kx = floor_log2_f32(scaled);
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
  const size_t nb = block_scales(n, block);
  double worst = 0.0;
  std::vector<float> x(static_cast<size_t>(block), 0.0f);
  for (size_t b = 0; b < nb; b++) {
    size_t base = b * size_t(block);
    float xmax = 0.0f;
    uint32_t vmax = 0;
    for (int j = 0; j < block; j++) {
      size_t i = base + size_t(j);
      if (i < n) {
        x[j] = v[i] - k[i];
        float ax = std::fabs(x[j]);
        if (ax > xmax) xmax = ax;
        uint32_t a = f32_bits(v[i]) & 0x7fffffffu;
        if (a > vmax) vmax = a;
      } else {
        x[j] = 0.0f;
      }
    }
    if (double(xmax) > worst) worst = double(xmax);
    int code = block_code(xmax, vmax, gate);
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
  return worst;
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

// ---------------------------------------------------------------------------------------------
// integer block frames
// ---------------------------------------------------------------------------------------------
int block_code_int(float xmax, uint32_t vmax_bits, const BlockGate& gate, int bits) {
  const uint32_t xb = f32_bits(xmax) & 0x7fffffffu;
  const int ef = int(xb >> 23);
  if (ef == 0 || ef == 255) return kSilent;       // zero, denormal, infinite or NaN
  const int ex = ef - 127;
  if (ex > 100) return kSilent;
  const uint32_t mant = xb & 0x7fffffu;
  // smallest exponent for which round(xmax / 2^e) <= 2^(bits-1) - 1
  int es = ex - (bits - 2);
  if (mant >= (1u << 23) - (1u << (24 - bits))) es += 1;
  if (es < gate.min_exp) es = gate.min_exp;
  if ((vmax_bits >> 23) != 0) {
    const int emax = int((vmax_bits >> 23) & 0xff) - 127;
    if (es < emax - gate.rel_bits) es = emax - gate.rel_bits;
  }
  if (es < kMinExp) es = kMinExp;
  // every element would round to zero: xmax <= 2^(es-1)
  if (ex < es - 1 || (ex == es - 1 && mant == 0)) return kSilent;
  return es + 127;
}

double encode_block_int(const float* v, float* k, size_t n, int block, const BlockGate& gate, int bits, uint8_t* codes,
                        uint8_t* scales) {
  const size_t nb = block_scales(n, block);
  const float M = 8388608.0f + float(1 << (bits - 1));
  const uint32_t mask = (1u << bits) - 1u;
  double worst = 0.0;
  for (size_t b = 0; b < nb; b++) {
    const size_t base = b * size_t(block);
    const size_t end = base + size_t(block) < n ? base + size_t(block) : n;
    float xmax = 0.0f;
    uint32_t vmax = 0;
    for (size_t i = base; i < end; i++) {
      float ax = std::fabs(v[i] - k[i]);
      if (ax > xmax) xmax = ax;
      uint32_t a = f32_bits(v[i]) & 0x7fffffffu;
      if (a > vmax) vmax = a;
    }
    if (double(xmax) > worst) worst = double(xmax);
    const int code = block_code_int(xmax, vmax, gate, bits);
    scales[b] = uint8_t(code);
    if (!code) {
      for (size_t i = base; i < end; i++) codes[i] = uint8_t(1u << (bits - 1));
      continue;
    }
    const float s = exp2i(code - 127), inv = exp2i(127 - code), neg_ms = -(M * s);
    for (size_t i = base; i < end; i++) {
      const float x = v[i] - k[i];
      const float z = std::fmaf(x, inv, M);
      codes[i] = uint8_t(f32_bits(z) & mask);
      k[i] += std::fmaf(z, s, neg_ms);
    }
  }
  return worst;
}

void block_int_steps(const uint8_t* codes, const uint8_t* scales, size_t n, int block, int bits, float* steps) {
  const size_t nb = block_scales(n, block);
  const float M = 8388608.0f + float(1 << (bits - 1));
  for (size_t b = 0; b < nb; b++) {
    const int code = scales[b];
    const size_t base = b * size_t(block);
    const size_t end = base + size_t(block) < n ? base + size_t(block) : n;
    if (code == 0 || code == 255) {
      for (size_t i = base; i < end; i++) steps[i] = 0.0f;
      continue;
    }
    const float s = exp2i(code - 127), neg_ms = -(M * s);
    for (size_t i = base; i < end; i++) steps[i] = std::fmaf(bits_f32(0x4b000000u | codes[i]), s, neg_ms);
  }
}

void decode_block_int_add(const uint8_t* codes, const uint8_t* scales, size_t n, int block, int bits, float sign, float* dst,
                          float* dst2) {
  const size_t nb = block_scales(n, block);
  const float M = 8388608.0f + float(1 << (bits - 1));
  for (size_t b = 0; b < nb; b++) {
    const int code = scales[b];
    if (code == 0 || code == 255) continue;
    const size_t base = b * size_t(block);
    const size_t end = base + size_t(block) < n ? base + size_t(block) : n;
    const float s = exp2i(code - 127), neg_ms = -(M * s);
    for (size_t i = base; i < end; i++) {
      const float step = sign * std::fmaf(bits_f32(0x4b000000u | codes[i]), s, neg_ms);
      dst[i] += step;
      if (dst2) dst2[i] += step;
    }
  }
}

void block_sign_steps(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* steps) {
  const size_t nb = block_scales(n, block);
  for (size_t b = 0; b < nb; b++) {
    const int code = scales[b];
    const size_t base = b * size_t(block);
    const size_t end = base + size_t(block) < n ? base + size_t(block) : n;
    const float s = (code == 0 || code == 255) ? 0.0f : exp2i(code - 127);
    for (size_t i = base; i < end; i++) steps[i] = s == 0.0f ? 0.0f : (((words[i >> 5] >> (i & 31)) & 1u) ? -s : s);
  }
}

void pack_tile_codes(const uint8_t* codes, int bits, uint32_t* out) {
  for (int w = 0; w < bits * 128; w++) out[w] = 0;
  const uint32_t mask = (1u << bits) - 1u;
  for (int i = 0; i < 4096; i++) {
    const int c = i >> 5, g = (i >> 2) & 7, e = i & 3;
    const int pos = c * 32 + ((g ^ (c & 7)) << 2) + e;   // position in the tile's code stream
    const int bit = pos * bits;
    out[bit >> 5] |= (uint32_t(codes[i]) & mask) << (bit & 31);
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
