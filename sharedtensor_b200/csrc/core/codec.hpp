// Sign-bit delta codec (host side).
//
// Two wire formats live here:
//
//  * tensor-scale frames: one fp32 scale followed by ceil(N/8) sign bytes, element i in byte i/8
//    bit i%8, bit 0 => +scale, bit 1 => -scale.  This is the format the reference speaks on its TCP
//    edges (reference src/sharedtensor.c:156-177 encoder, 106-111 decoder) and is reproduced
//    bit for bit, including "zero counts as negative" (168-172) and scale==0 no-op frames.
//
//  * block-scale frames: one E8M0-style exponent byte per block of B elements (B a power of two,
//    32..4096) plus one 32-bit sign word per 32 elements (bit j of word w = element 32*w+j, so the
//    little-endian byte stream has the same bit order as the tensor-scale frame).  This is the
//    format the GPU kernels produce and consume; the functions here are their bit-exact CPU oracle.
//
// State model ("mirror form").  A replica keeps its values V and, per edge e, a mirror K_e = the
// part of V that the neighbour on e is already known to hold (everything sent to it plus everything
// received from it).  The quantity the reference calls the edge residual (`Connection.delta`,
// src/sharedtensor.c:27) is V - K_e, so encoding is "quantise V - K_e, add the quantised step to
// K_e", and decoding a frame from e is "add the step to V and to K_e".  Updates received on another
// edge change V but not K_e, which forwards them, exactly like src/sharedtensor.c:124-127.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace st {

// ---------------------------------------------------------------------------------------------
// Exponent helpers shared (by construction, not by include) with the CUDA kernels.
// ---------------------------------------------------------------------------------------------

// Code 0 means "silent block": nothing is applied for that block in this frame.
constexpr int kSilent = 0;
// Smallest / largest exponent a code can carry: code = exponent + 127, codes 1..254.
constexpr int kMinExp = -126;
constexpr int kMaxExp = 127;

inline uint32_t f32_bits(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  return u;
}
inline float bits_f32(uint32_t u) {
  float x;
  std::memcpy(&x, &u, 4);
  return x;
}

// floor(log2(x)) for a finite positive normal fp32 x, taken from the exponent field; for zero and
// denormals returns -127 (callers treat anything that small as silent).
inline int floor_log2_f32(float x) { return int((f32_bits(x) >> 23) & 0xff) - 127; }

// 2^k as fp32 for k in [-126, 127].
inline float exp2i(int k) { return bits_f32(uint32_t(k + 127) << 23); }

struct BlockGate {
  int min_exp = -100;  // blocks whose scale exponent is below this stay silent
  int rel_bits = 22;   // ... or below (exponent of the block's largest |value|) - rel_bits
};

// ---------------------------------------------------------------------------------------------
// Tensor-scale (reference wire format)
// ---------------------------------------------------------------------------------------------

size_t sign_bytes(size_t n);  // ceil(n/8)

// Power-of-two floor of the RMS of r[0..n), summed left to right in fp32 like the reference
// (src/sharedtensor.c:156-159).  Returns 0 for an all-zero (or underflowing) input.
float ref_scale_of(const float* r, size_t n);

// Reference encoder on an explicit residual array (src/sharedtensor.c:166-174): chooses the scale,
// writes the sign bytes, moves every residual element by -/+ scale.  Returns the scale.
float encode_residual_ref(float* r, size_t n, uint8_t* bits);

// Mirror-form encoder: quantises v - k with one scale for the whole tensor, adds the step to k.
// `min_scale`: if the chosen scale is below it the frame is a no-op (scale 0, k untouched).
// `rule`: 0 = the reference's scale (power-of-two floor of the RMS), 1 = bisection (power-of-two floor of 2/3 of
// the largest residual; the error bound halves with every frame).
// Returns the scale written on the wire.
float encode_tensor(const float* v, float* k, size_t n, uint8_t* bits, float min_scale, int rule = 1);

// Decoder: dst[i] += (bit ? -scale : +scale).  `dst2` may be null; if not it gets the same step.
void decode_tensor_add(const uint8_t* bits, float scale, size_t n, float* dst, float* dst2);

// Fast paths (codec_fast.cpp): AVX2 where the CPU has it, several threads for large tensors; bit-for-bit the
// results of the plain functions above.  encode_tensor_fast is rule 1 (bisection) with the smallest useful
// scale given as max(min_scale_abs, min_scale_rel * max|v|), found in the same pass as the largest residual.
float encode_tensor_fast(const float* v, float* k, size_t n, uint8_t* bits, float min_scale_abs, float min_scale_rel);
void decode_tensor_add_fast(const uint8_t* bits, float scale, size_t n, float* dst, float* dst2);
void add_fast(float* values, const float* delta, size_t n);
void sub_add_fast(float* values, const float* neu, const float* old, size_t n);
void copy_fast(float* dst, const float* src, size_t n);

// ---------------------------------------------------------------------------------------------
// Block-scale (GPU format; CPU oracle)
// ---------------------------------------------------------------------------------------------

size_t block_words(size_t n);              // ceil(n/32)
size_t block_scales(size_t n, int block);  // ceil(n/block)

// Exponent code of one block from its largest |residual| and the bit pattern of its largest |value| (0 = silent).
int block_code(float xmax, uint32_t vmax_bits, const BlockGate& gate);

// Encodes n elements (n need not be a multiple of anything; missing elements count as zero residual
// and their bits are 1).  v: values, k: mirror (updated), words/scales: outputs.
// Returns the largest |residual| (before the update), a cheap convergence statistic.
double encode_block(const float* v, float* k, size_t n, int block, const BlockGate& gate,
                    uint32_t* words, uint8_t* scales);

// Applies one block-scale frame to dst (and dst2 if non-null).
void decode_block_add(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* dst,
                      float* dst2);
// The same two, cut into block-aligned pieces over several threads for large tensors.
double encode_block_fast(const float* v, float* k, size_t n, int block, const BlockGate& gate, uint32_t* words,
                         uint8_t* scales);
void decode_block_add_fast(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* dst, float* dst2);

// ---------------------------------------------------------------------------------------------
// Integer block frames (GPU rings with 2, 4 or 8 bits per element; CPU oracle)
//
// One exponent byte per block (as above) and one `bits`-bit integer per element: the block's residuals
// x = v - k are rounded to the nearest multiple of the block's step 2^e (ties to even) and the multiple m,
// |m| <= 2^(bits-1) - 1, travels as m + 2^(bits-1).  The step is the smallest power of two for which the
// block's largest residual still fits, but never below the cut-off of BlockGate, so one frame takes the
// largest residual of a block down by a factor of about 2^(bits-1): 8-bit frames bring a fresh update to
// under one percent in a single frame where sign frames (the reference's 1 bit per element,
// src/sharedtensor.c:166-174) need about ten.  A residual of zero is the code of zero: elements that have
// nothing to say do not move.  The arithmetic is spelled out so that the kernels (../cuda/round.cu) and this
// file agree bit for bit:
//   z = fma(x, 2^-e, M)   with M = 2^23 + 2^(bits-1)      (the low bits of z's mantissa are the code)
//   step = fma(z, 2^e, -(M * 2^e))                         (exact: (z - M) * 2^e)
//   k += step
// Residuals at or above 2^101 are not sent (the block stays silent): M * 2^e must not overflow.
// ---------------------------------------------------------------------------------------------

// Exponent code (0 = silent) of a block from its largest |residual| and the bits of its largest |value|.
int block_code_int(float xmax, uint32_t vmax_bits, const BlockGate& gate, int bits);

// Encodes n elements into one code byte per element (unpacked; the low `bits` bits are used) and one scale
// byte per block; steps the mirror.  Returns the largest |residual| before the update.
double encode_block_int(const float* v, float* k, size_t n, int block, const BlockGate& gate, int bits, uint8_t* codes,
                        uint8_t* scales);

// The step every element receives from one frame (0 where the block is silent), for integer frames
// (bits = 2, 4, 8; `codes` one byte per element) ...
void block_int_steps(const uint8_t* codes, const uint8_t* scales, size_t n, int block, int bits, float* steps);
// ... and for sign frames (`words` as produced by encode_block).
void block_sign_steps(const uint32_t* words, const uint8_t* scales, size_t n, int block, float* steps);

// Adds sign * (the steps of one integer frame) to dst and, if given, dst2 (sign = +1 applies a frame, -1 takes it back).
void decode_block_int_add(const uint8_t* codes, const uint8_t* scales, size_t n, int block, int bits, float sign, float* dst,
                          float* dst2);
// 8-bit integer frames with one code byte per element, as TCP edges between nodes of this framework can carry them
// (AVX2 + FMA and several threads where available; bit for bit what encode_block_int / decode_block_int_add give).
double encode_block_int8_fast(const float* v, float* k, size_t n, int block, const BlockGate& gate, uint8_t* codes,
                              uint8_t* scales);
void decode_block_int8_add_fast(const uint8_t* codes, const uint8_t* scales, size_t n, int block, float sign, float* dst,
                                float* dst2);

// Layout of one tile (4096 elements) in a GPU ring slot: `bits` * 128 words of codes, then the scale bytes.
// Codes are packed little-endian, `bits` per element, in the order the kernel's threads hold them: within
// the c-th run of 32 elements the g-th group of four elements sits at position g ^ (c & 7).  `codes` holds
// 4096 unpacked codes (for sign frames: 0 or 1), `out` receives bits * 128 words.
void pack_tile_codes(const uint8_t* codes, int bits, uint32_t* out);

// Per-segment sum of squares over a flat arena (table sync; README.md:41 of the reference lists
// per-tensor magnitudes as a TODO).  offsets has n_seg+1 entries.
void segment_sumsq(const float* x, const int64_t* offsets, int n_seg, double* out);

}  // namespace st
