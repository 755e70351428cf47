// Fast host paths of the tensor-scale codec and of the element-wise replica updates: AVX2 where the CPU has it
// (checked at run time), several threads for large tensors.  Every function here produces bit-for-bit what its
// plain counterpart in codec.cpp produces — same per-element operations, order-independent reductions (maxima) —
// and the tests hold them to that.  The reference does all of this in scalar loops on the calling thread
// (src/sharedtensor.c:156-174 encode, 106-111 decode, 448-453 add).
#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "codec.hpp"

namespace st {

namespace {

int max_threads() {
  static const int v = [] {
    int hw = int(std::thread::hardware_concurrency());
    if (hw < 1) hw = 1;
    int t = hw > 8 ? 8 : hw;
    if (const char* e = std::getenv("SHAREDTENSOR_CPU_THREADS")) {
      int x = std::atoi(e);
      if (x >= 1 && x <= 64) t = x;
    }
    return t;
  }();
  return v;
}

bool have_avx2() {
  static const bool v = __builtin_cpu_supports("avx2");
  return v;
}

// Runs fn(begin, end) over [0, n) cut into at most max_threads() pieces whose boundaries are multiples of `align`.
template <class F>
void parallel_chunks(size_t n, size_t align, F fn) {
  constexpr size_t kGrain = size_t(1) << 19;  // below this a second thread costs more than it saves
  size_t t = std::min<size_t>(size_t(max_threads()), n / kGrain);
  if (t <= 1) {
    fn(size_t(0), n, 0);
    return;
  }
  size_t chunk = (n + t - 1) / t;
  chunk = (chunk + align - 1) / align * align;
  std::vector<std::thread> th;
  th.reserve(t - 1);
  int idx = 1;
  for (size_t b = chunk; b < n; b += chunk, idx++) {
    size_t e = std::min(n, b + chunk);
    th.emplace_back([=] { fn(b, e, idx); });
  }
  fn(size_t(0), std::min(n, chunk), 0);
  for (auto& x : th) x.join();
}

// ---- maxima of |v| and |v - k| ------------------------------------------------------------------
void maxabs2_scalar(const float* v, const float* k, size_t b, size_t e, float* vmax, float* xmax) {
  float a = 0.0f, x = 0.0f;
  for (size_t i = b; i < e; i++) {
    float av = std::fabs(v[i]);
    if (av > a) a = av;
    float ax = std::fabs(v[i] - k[i]);
    if (ax > x) x = ax;
  }
  *vmax = a;
  *xmax = x;
}

__attribute__((target("avx2"))) void maxabs2_avx2(const float* v, const float* k, size_t b, size_t e, float* vmax,
                                                  float* xmax) {
  const __m256 absmask = _mm256_castsi256_ps(_mm256_set1_epi32(0x7fffffff));
  __m256 a = _mm256_setzero_ps(), x = _mm256_setzero_ps();
  size_t i = b;
  for (; i + 8 <= e; i += 8) {
    __m256 vv = _mm256_loadu_ps(v + i);
    __m256 kk = _mm256_loadu_ps(k + i);
    // max_ps(new, acc) returns acc when new is NaN: the same as the scalar "if (new > acc)"
    a = _mm256_max_ps(_mm256_and_ps(vv, absmask), a);
    x = _mm256_max_ps(_mm256_and_ps(_mm256_sub_ps(vv, kk), absmask), x);
  }
  float ta[8], tx[8];
  _mm256_storeu_ps(ta, a);
  _mm256_storeu_ps(tx, x);
  float ra = 0.0f, rx = 0.0f;
  for (int j = 0; j < 8; j++) {
    if (ta[j] > ra) ra = ta[j];
    if (tx[j] > rx) rx = tx[j];
  }
  float sa, sx;
  maxabs2_scalar(v, k, i, e, &sa, &sx);
  *vmax = sa > ra ? sa : ra;
  *xmax = sx > rx ? sx : rx;
}

// ---- sign bits and mirror step ------------------------------------------------------------------
// [b, e) with b a multiple of 8; writes bits[b/8 ...]
void sign_step_scalar(const float* v, float* k, size_t b, size_t e, uint8_t* bits, float scale) {
  for (size_t i = b; i < e; i += 8) {
    unsigned byte = 0;
    size_t lim = std::min(e, i + 8);
    for (size_t j = i; j < lim; j++) {
      float x = v[j] - k[j];
      if (x > 0.0f) {
        k[j] += scale;
      } else {
        byte |= 1u << (j - i);
        k[j] -= scale;
      }
    }
    bits[i >> 3] = uint8_t(byte);
  }
}

__attribute__((target("avx2"))) void sign_step_avx2(const float* v, float* k, size_t b, size_t e, uint8_t* bits,
                                                    float scale) {
  const __m256 zero = _mm256_setzero_ps();
  const __m256 pos = _mm256_set1_ps(scale), neg = _mm256_set1_ps(-scale);
  size_t i = b;
  for (; i + 8 <= e; i += 8) {
    __m256 vv = _mm256_loadu_ps(v + i);
    __m256 kk = _mm256_loadu_ps(k + i);
    __m256 gt = _mm256_cmp_ps(_mm256_sub_ps(vv, kk), zero, _CMP_GT_OQ);  // x > 0, false for NaN like the scalar test
    bits[i >> 3] = uint8_t(~unsigned(_mm256_movemask_ps(gt)) & 0xffu);
    _mm256_storeu_ps(k + i, _mm256_add_ps(kk, _mm256_blendv_ps(neg, pos, gt)));
  }
  if (i < e) sign_step_scalar(v, k, i, e, bits, scale);
}

// scale-0 frame: bits only, the mirror does not move
void sign_only(const float* v, const float* k, size_t b, size_t e, uint8_t* bits) {
  for (size_t i = b; i < e; i += 8) {
    unsigned byte = 0;
    size_t lim = std::min(e, i + 8);
    for (size_t j = i; j < lim; j++)
      if (!(v[j] - k[j] > 0.0f)) byte |= 1u << (j - i);
    bits[i >> 3] = uint8_t(byte);
  }
}

// ---- decode ---------------------------------------------------------------------------------------
void decode_scalar(const uint8_t* bits, float scale, size_t b, size_t e, float* dst, float* dst2) {
  const float step[2] = {scale, -scale};
  for (size_t i = b; i < e; i++) {
    float f = step[(bits[i >> 3] >> (i & 7)) & 1];
    dst[i] += f;
    if (dst2) dst2[i] += f;
  }
}

__attribute__((target("avx2"))) void decode_avx2(const uint8_t* bits, float scale, size_t b, size_t e, float* dst,
                                                 float* dst2) {
  const __m256i lane_bit = _mm256_setr_epi32(1, 2, 4, 8, 16, 32, 64, 128);
  const __m256 pos = _mm256_set1_ps(scale), neg = _mm256_set1_ps(-scale);
  size_t i = b;  // b is a multiple of 8
  for (; i + 8 <= e; i += 8) {
    __m256i byte = _mm256_set1_epi32(int(bits[i >> 3]));
    __m256 isneg = _mm256_castsi256_ps(_mm256_cmpeq_epi32(_mm256_and_si256(byte, lane_bit), lane_bit));
    __m256 f = _mm256_blendv_ps(pos, neg, isneg);
    _mm256_storeu_ps(dst + i, _mm256_add_ps(_mm256_loadu_ps(dst + i), f));
    if (dst2) _mm256_storeu_ps(dst2 + i, _mm256_add_ps(_mm256_loadu_ps(dst2 + i), f));
  }
  if (i < e) decode_scalar(bits, scale, i, e, dst, dst2);
}

float pow2_floor_f(float s) {
  if (!(s > 0.0f) || std::isinf(s)) return 0.0f;
  int e;
  std::frexp(double(s), &e);
  return float(std::ldexp(1.0, e - 1));
}

}  // namespace

float encode_tensor_fast(const float* v, float* k, size_t n, uint8_t* bits, float min_scale_abs, float min_scale_rel) {
  const bool avx = have_avx2();
  float vmaxs[64], xmaxs[64];
  for (int i = 0; i < 64; i++) vmaxs[i] = xmaxs[i] = 0.0f;
  parallel_chunks(n, 8, [&](size_t b, size_t e, int idx) {
    if (avx) maxabs2_avx2(v, k, b, e, &vmaxs[idx], &xmaxs[idx]);
    else maxabs2_scalar(v, k, b, e, &vmaxs[idx], &xmaxs[idx]);
  });
  float vmax = 0.0f, xmax = 0.0f;
  for (int i = 0; i < 64; i++) {
    if (vmaxs[i] > vmax) vmax = vmaxs[i];
    if (xmaxs[i] > xmax) xmax = xmaxs[i];
  }
  float min_scale = min_scale_abs;
  if (min_scale_rel > 0.0f) {
    float rel = vmax * min_scale_rel;
    if (rel > min_scale) min_scale = rel;
  }
  float scale = pow2_floor_f(xmax * 0.6666667f);
  if (scale < min_scale) scale = 0.0f;
  if (scale == 0.0f) {
    parallel_chunks(n, 8, [&](size_t b, size_t e, int) { sign_only(v, k, b, e, bits); });
    return 0.0f;
  }
  parallel_chunks(n, 8, [&](size_t b, size_t e, int) {
    if (avx) sign_step_avx2(v, k, b, e, bits, scale);
    else sign_step_scalar(v, k, b, e, bits, scale);
  });
  return scale;
}

void decode_tensor_add_fast(const uint8_t* bits, float scale, size_t n, float* dst, float* dst2) {
  if (scale == 0.0f) return;
  const bool avx = have_avx2();
  parallel_chunks(n, 8, [&](size_t b, size_t e, int) {
    if (avx) decode_avx2(bits, scale, b, e, dst, dst2);
    else decode_scalar(bits, scale, b, e, dst, dst2);
  });
}

void add_fast(float* values, const float* delta, size_t n) {
  parallel_chunks(n, 16, [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; i++) values[i] += delta[i];
  });
}

void sub_add_fast(float* values, const float* neu, const float* old, size_t n) {
  parallel_chunks(n, 16, [&](size_t b, size_t e, int) {
    for (size_t i = b; i < e; i++) values[i] += neu[i] - old[i];
  });
}

void copy_fast(float* dst, const float* src, size_t n) {
  parallel_chunks(n, 16, [&](size_t b, size_t e, int) { std::memcpy(dst + b, src + b, (e - b) * sizeof(float)); });
}

namespace {

// Full blocks only (n a multiple of `block`, block a multiple of 32); same results as encode_block.
__attribute__((target("avx2"))) double encode_blocks_avx2(const float* v, float* k, size_t n, int block, const BlockGate& gate,
                                                          uint32_t* words, uint8_t* scales) {
  const __m256 absmask = _mm256_castsi256_ps(_mm256_set1_epi32(0x7fffffff));
  const __m256 zero = _mm256_setzero_ps();
  double worst = 0.0;
  const size_t nb = n / size_t(block);
  for (size_t b = 0; b < nb; b++) {
    const float* vb = v + b * size_t(block);
    float* kb = k + b * size_t(block);
    __m256 xm = _mm256_setzero_ps();
    __m256i vm = _mm256_setzero_si256();
    for (int j = 0; j < block; j += 8) {
      const __m256 vv = _mm256_loadu_ps(vb + j);
      const __m256 x = _mm256_sub_ps(vv, _mm256_loadu_ps(kb + j));
      xm = _mm256_max_ps(_mm256_and_ps(x, absmask), xm);  // a NaN residual is skipped, like "if (ax > xmax)"
      vm = _mm256_max_epu32(vm, _mm256_castps_si256(_mm256_and_ps(vv, absmask)));
    }
    float tx[8];
    uint32_t tv[8];
    _mm256_storeu_ps(tx, xm);
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(tv), vm);
    float xmax = 0.0f;
    uint32_t vmax = 0;
    for (int j = 0; j < 8; j++) {
      if (tx[j] > xmax) xmax = tx[j];
      if (tv[j] > vmax) vmax = tv[j];
    }
    if (double(xmax) > worst) worst = double(xmax);
    const int code = block_code(xmax, vmax, gate);
    scales[b] = uint8_t(code);
    const float scale = code ? exp2i(code - 127) : 0.0f;
    const __m256 pos = _mm256_set1_ps(scale), neg = _mm256_set1_ps(-scale);
    uint32_t* wb = words + b * size_t(block / 32);
    for (int g = 0; g < block / 32; g++) {
      uint32_t w = 0;
      for (int j = 0; j < 32; j += 8) {
        const int o = g * 32 + j;
        const __m256 kk = _mm256_loadu_ps(kb + o);
        const __m256 gt = _mm256_cmp_ps(_mm256_sub_ps(_mm256_loadu_ps(vb + o), kk), zero, _CMP_GT_OQ);
        w |= (~uint32_t(_mm256_movemask_ps(gt)) & 0xffu) << j;
        if (code) _mm256_storeu_ps(kb + o, _mm256_add_ps(kk, _mm256_blendv_ps(neg, pos, gt)));
      }
      wb[g] = w;
    }
  }
  return worst;
}

__attribute__((target("avx2"))) void decode_blocks_avx2(const uint32_t* words, const uint8_t* scales, size_t n, int block,
                                                        float* dst, float* dst2) {
  const __m256i lane_bit = _mm256_setr_epi32(1, 2, 4, 8, 16, 32, 64, 128);
  const size_t nb = n / size_t(block);
  for (size_t b = 0; b < nb; b++) {
    const int code = scales[b];
    if (!code) continue;
    const float scale = exp2i(code - 127);
    const __m256 pos = _mm256_set1_ps(scale), neg = _mm256_set1_ps(-scale);
    const size_t base = b * size_t(block);
    for (int j = 0; j < block; j += 8) {
      const size_t i = base + size_t(j);
      const __m256i byte = _mm256_set1_epi32(int((words[i >> 5] >> (i & 31)) & 0xffu));
      const __m256 isneg = _mm256_castsi256_ps(_mm256_cmpeq_epi32(_mm256_and_si256(byte, lane_bit), lane_bit));
      const __m256 f = _mm256_blendv_ps(pos, neg, isneg);
      _mm256_storeu_ps(dst + i, _mm256_add_ps(_mm256_loadu_ps(dst + i), f));
      if (dst2) _mm256_storeu_ps(dst2 + i, _mm256_add_ps(_mm256_loadu_ps(dst2 + i), f));
    }
  }
}

// ---- 8-bit integer frames, full blocks only (block a multiple of 32) ----
__attribute__((target("avx2,fma"))) double encode_blocks_int8_avx2(const float* v, float* k, size_t n, int block,
                                                                   const BlockGate& gate, uint8_t* codes, uint8_t* scales) {
  const __m256 absmask = _mm256_castsi256_ps(_mm256_set1_epi32(0x7fffffff));
  const __m256i bytemask = _mm256_set1_epi32(0xff);
  const __m256i order = _mm256_setr_epi32(0, 4, 1, 5, 2, 6, 3, 7);
  const float M = 8388608.0f + 128.0f;
  const __m256 vM = _mm256_set1_ps(M);
  double worst = 0.0;
  const size_t nb = n / size_t(block);
  for (size_t b = 0; b < nb; b++) {
    const float* vb = v + b * size_t(block);
    float* kb = k + b * size_t(block);
    uint8_t* cb = codes + b * size_t(block);
    __m256 xm = _mm256_setzero_ps();
    __m256i vm = _mm256_setzero_si256();
    for (int j = 0; j < block; j += 8) {
      const __m256 vv = _mm256_loadu_ps(vb + j);
      const __m256 x = _mm256_sub_ps(vv, _mm256_loadu_ps(kb + j));
      xm = _mm256_max_ps(_mm256_and_ps(x, absmask), xm);
      vm = _mm256_max_epu32(vm, _mm256_castps_si256(_mm256_and_ps(vv, absmask)));
    }
    float tx[8];
    uint32_t tv[8];
    _mm256_storeu_ps(tx, xm);
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(tv), vm);
    float xmax = 0.0f;
    uint32_t vmax = 0;
    for (int j = 0; j < 8; j++) {
      if (tx[j] > xmax) xmax = tx[j];
      if (tv[j] > vmax) vmax = tv[j];
    }
    if (double(xmax) > worst) worst = double(xmax);
    const int code = block_code_int(xmax, vmax, gate, 8);
    scales[b] = uint8_t(code);
    if (!code) {
      std::memset(cb, 0x80, size_t(block));
      continue;
    }
    const float s = exp2i(code - 127);
    const __m256 vs = _mm256_set1_ps(s), vinv = _mm256_set1_ps(exp2i(127 - code)), vneg = _mm256_set1_ps(-(M * s));
    for (int j = 0; j < block; j += 32) {
      __m256i zb[4];
      for (int q = 0; q < 4; q++) {
        const int o = j + q * 8;
        const __m256 kk = _mm256_loadu_ps(kb + o);
        const __m256 z = _mm256_fmadd_ps(_mm256_sub_ps(_mm256_loadu_ps(vb + o), kk), vinv, vM);
        zb[q] = _mm256_and_si256(_mm256_castps_si256(z), bytemask);
        _mm256_storeu_ps(kb + o, _mm256_add_ps(kk, _mm256_fmadd_ps(z, vs, vneg)));
      }
      // 4 x 8 values below 256 -> 32 bytes in element order (the packs work within 128-bit halves)
      const __m256i p = _mm256_packus_epi16(_mm256_packus_epi32(zb[0], zb[1]), _mm256_packus_epi32(zb[2], zb[3]));
      _mm256_storeu_si256(reinterpret_cast<__m256i*>(cb + j), _mm256_permutevar8x32_epi32(p, order));
    }
  }
  return worst;
}

__attribute__((target("avx2,fma"))) void decode_blocks_int8_avx2(const uint8_t* codes, const uint8_t* scales, size_t n,
                                                                 int block, float sign, float* dst, float* dst2) {
  const float M = 8388608.0f + 128.0f;
  const __m256i expo = _mm256_set1_epi32(0x4b000000);
  const __m256 vsign = _mm256_set1_ps(sign);
  const size_t nb = n / size_t(block);
  for (size_t b = 0; b < nb; b++) {
    const int code = scales[b];
    if (code == 0 || code == 255) continue;
    const float s = exp2i(code - 127);
    const __m256 vs = _mm256_set1_ps(s), vneg = _mm256_set1_ps(-(M * s));
    const size_t base = b * size_t(block);
    for (int j = 0; j < block; j += 8) {
      const size_t i = base + size_t(j);
      const __m256i c = _mm256_cvtepu8_epi32(_mm_loadl_epi64(reinterpret_cast<const __m128i*>(codes + i)));
      const __m256 step = _mm256_mul_ps(vsign, _mm256_fmadd_ps(_mm256_castsi256_ps(_mm256_or_si256(c, expo)), vs, vneg));
      _mm256_storeu_ps(dst + i, _mm256_add_ps(_mm256_loadu_ps(dst + i), step));
      if (dst2) _mm256_storeu_ps(dst2 + i, _mm256_add_ps(_mm256_loadu_ps(dst2 + i), step));
    }
  }
}

bool have_fma() {
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return ok;
}

}  // namespace

double encode_block_int8_fast(const float* v, float* k, size_t n, int block, const BlockGate& gate, uint8_t* codes,
                              uint8_t* scales) {
  const bool avx = have_fma();
  double worst[64];
  for (int i = 0; i < 64; i++) worst[i] = 0.0;
  parallel_chunks(n, size_t(block), [&](size_t b, size_t e, int idx) {
    const size_t full = avx ? (e - b) / size_t(block) * size_t(block) : 0;
    double w = 0.0;
    if (full) w = encode_blocks_int8_avx2(v + b, k + b, full, block, gate, codes + b, scales + b / size_t(block));
    if (b + full < e) {
      const size_t o = b + full;
      double w2 = encode_block_int(v + o, k + o, e - o, block, gate, 8, codes + o, scales + o / size_t(block));
      if (w2 > w) w = w2;
    }
    worst[idx] = w;
  });
  double w = 0.0;
  for (int i = 0; i < 64; i++)
    if (worst[i] > w) w = worst[i];
  return w;
}

void decode_block_int8_add_fast(const uint8_t* codes, const uint8_t* scales, size_t n, int block, float sign, float* dst,
                                float* dst2) {
  const bool avx = have_fma();
  parallel_chunks(n, size_t(block), [&](size_t b, size_t e, int) {
    const size_t full = avx ? (e - b) / size_t(block) * size_t(block) : 0;
    if (full) decode_blocks_int8_avx2(codes + b, scales + b / size_t(block), full, block, sign, dst + b, dst2 ? dst2 + b : nullptr);
    if (b + full < e) {
      const size_t o = b + full;
      decode_block_int_add(codes + o, scales + o / size_t(block), e - o, block, 8, sign, dst + o, dst2 ? dst2 + o : nullptr);
    }
  });
}

double encode_block_fast(const float* v, float* k, size_t n, int block, const BlockGate& gate, uint32_t* words,
                         uint8_t* scales) {
  const bool avx = have_avx2();
  double worst[64];
  for (int i = 0; i < 64; i++) worst[i] = 0.0;
  parallel_chunks(n, size_t(block), [&](size_t b, size_t e, int idx) {
    const size_t full = avx ? (e - b) / size_t(block) * size_t(block) : 0;  // whole blocks go through AVX2
    double w = 0.0;
    if (full) w = encode_blocks_avx2(v + b, k + b, full, block, gate, words + b / 32, scales + b / size_t(block));
    if (b + full < e) {
      const size_t o = b + full;
      double w2 = encode_block(v + o, k + o, e - o, block, gate, words + o / 32, scales + o / size_t(block));
      if (w2 > w) w = w2;
    }
    worst[idx] = w;
  });
  double w = 0.0;
  for (int i = 0; i < 64; i++)
    if (worst[i] > w) w = worst[i];
  return w;
}

void decode_block_add_fast(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* dst, float* dst2) {
  const bool avx = have_avx2();
  parallel_chunks(n, size_t(block), [&](size_t b, size_t e, int) {
    const size_t full = avx ? (e - b) / size_t(block) * size_t(block) : 0;
    if (full) decode_blocks_avx2(words + b / 32, scales + b / size_t(block), full, block, dst + b, dst2 ? dst2 + b : nullptr);
    if (b + full < e) {
      const size_t o = b + full;
      decode_block_add(words + o / 32, scales + o / size_t(block), e - o, block, dst + o, dst2 ? dst2 + o : nullptr);
    }
  });
}

}  // namespace st
