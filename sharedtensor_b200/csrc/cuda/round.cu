// The sync-round kernel for sm_100a (see round.h for the protocol and ../core/codec.hpp for the arithmetic).
//
// A CTA holds up to three independent groups and one publisher warp; a group is four compute warps and one I/O warp
// and owns every n-th tile of the tensor.  The kinds of warp talk through shared memory and mbarriers only:
//
//   I/O warp      reads its tiles' sequence flags, credits and change marks (32 tiles at a time, one per lane),
//                 and for every tile with something to do hands the compute warps one *step* per link: it writes
//                 the step's descriptor (tile, link, which frames arrived, which rings have room), and stages the
//                 tile's values and the link's mirror into a slot with 1-D TMA bulk copies (cp.async.bulk,
//                 completion on the slot's `full` mbarrier; every source is this GPU's own memory).  When the
//                 compute warps have finished a step (`done` mbarrier) it issues the step's bulk stores straight
//                 from the slot: the decoded frames as a bulk reduce-add into the values (so an update another
//                 stream adds at the same moment is never overwritten), the stepped mirror, and the packed codes
//                 and scale bytes into the ring slot of every neighbour on the link (peer stores over NVLink;
//                 reference src/sharedtensor.c:176-177, two socket writes).  Two steps later, when those stores
//                 have completed, it hands the step to the publisher warp.
//   publisher     one warp per CTA: takes the completed steps of all groups, executes the system-scope fence (which
//                 costs microseconds, and would otherwise stall an I/O warp) and writes sequence flags to the
//                 receivers and credits to the senders, one ring per lane.
//   compute warps a thread owns 32 consecutive elements of the tile (read from shared memory through an XOR
//                 swizzle, so no bank conflicts).  It decodes the frames that arrived (reference 106-111, 124-127)
//                 into one accumulated step, adds it to its values and to the mirror of the link the frames came
//                 from, then forms values - mirror, the block's largest magnitude, the exponent code, the codes
//                 of its 32 elements, and steps the mirror by what the codes say (reference 156-174).
//
// Nothing in here waits for another GPU.  The waits are on this CTA's own copies and on its own warps, and every
// one is bounded: when a wait runs out the group records an error in the status block, stores nothing of the step
// it was on, marks its tiles for another visit and leaves.
//
// Arithmetic is written with explicit round-to-nearest operations; block statistics are maxima (order does not
// matter), so codes, scales, mirrors and values are bit-identical to the host codec (../core/codec.cpp).
#include <cuda_runtime.h>

#include <cstdint>

#include "round.h"

#ifdef ST_ROUND_DEBUG
// progress marks in host memory, readable while a kernel is stuck (debug builds only)
#define ST_CRUMB(slot, code)                                                                  \
  do {                                                                                         \
    if (p.dbg != nullptr && lane == 0) {                                                       \
      *reinterpret_cast<volatile uint32_t*>(p.dbg + (blockIdx.x * 8 + (slot))) = uint32_t(code); \
    }                                                                                          \
  } while (0)
#else
#define ST_CRUMB(slot, code)
#endif
#ifdef ST_ROUND_TIMELINE
// time stamps (ns, low 32 bits) of the first steps of CTA 0 / group 0 in the debug buffer: [1024 + step * 8 + event]
#define ST_STAMP(step, ev)                                                                                   \
  do {                                                                                                       \
    if (p.dbg != nullptr && blockIdx.x == 0 && g == 0 && lane == 0 && (step) < 24u)                          \
      *reinterpret_cast<volatile uint32_t*>(p.dbg + 1024 + (step) * 8 + (ev)) = uint32_t(globaltimer_ns()); \
  } while (0)
#else
#define ST_STAMP(step, ev)
#endif
#ifdef ST_ROUND_TIMING
#include <cstdio>
#define ST_T0() const long long st_t0_ = clock64()
#define ST_ACC(var) var += clock64() - st_t0_
#define ST_LAP(var) { const long long st_now_ = clock64(); var += st_now_ - st_lap_; st_lap_ = st_now_; }
#else
#define ST_T0()
#define ST_ACC(var)
#define ST_LAP(var)
#endif

namespace st {

namespace {

constexpr int kGroupThreads = 128;  // compute threads of a group: one per 32 consecutive elements of a tile
constexpr int kTileBytes = kTile * 4;
constexpr int kPubQueue = 32;
// Shapes of a CTA (groups x staging slots per group); the launcher picks one, see launch_round.
//   3 x 2: one CTA per SM, 12 compute warps                (fills the SM's shared memory and registers)
//   2 x 3: one CTA per SM,  8 compute warps, deeper staging (leaves a third of the registers to other kernels)
// Either way a group takes every n-th tile of the tensor for the whole launch, or (RoundParams::chunk) a run of
// consecutive tiles, in which case the grid has many short-lived CTAs and other kernels get SMs in between.

// ----------------------------------------------------------------------------------------------
// small PTX wrappers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// this GPU's own bookkeeping words, written and read by different lanes and launches: always at the L2
__device__ __forceinline__ uint32_t ld_cg_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_cg_u32(uint32_t* p, uint32_t v) { asm volatile("st.global.cg.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
// frame words and scale bytes were written by a neighbour GPU: read them from the L2, never from this SM's L1
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_cg_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_cg_word(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_cg_u8(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`.  Source is always local
// device memory; size and both addresses are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// shared -> global bulk store / reduce (this CTA's memory as source), tracked by bulk async-groups
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_f32(float* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all_but_2() { asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_shared_volatile(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }
__device__ __forceinline__ void st_shared_volatile(uint32_t* p, uint32_t v) { *reinterpret_cast<volatile uint32_t*>(p) = v; }

// Bounded wait on one of this CTA's own barriers; false when `limit_ns` has passed.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < (1u << 26); it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 15) == 15 && globaltimer_ns() - t0 > limit_ns) return false;
  }
  return false;
}

// A compute warp's wait for the descriptor of a step.  While the I/O warp looks for work, or there is none, a compute
// warp may sit here for the whole launch, so the limit is generous; it only covers an I/O warp that never comes back.
__device__ __forceinline__ bool wait_armed(const uint32_t* armed, uint32_t step, const uint32_t* abort) {
  if (ld_shared_volatile(armed) > step) return true;
  const uint64_t t_start = globaltimer_ns();
  for (uint32_t it = 0; it < (1u << 28); it++) {
    if (ld_shared_volatile(armed) > step) return true;
    if (ld_shared_volatile(abort)) return false;
    if ((it & 63) == 63 && globaltimer_ns() - t_start > 2000ull * 1000 * 1000) return false;
    __nanosleep(20);
  }
  return false;
}

// ----------------------------------------------------------------------------------------------
// what the I/O warp tells the compute warps about a step (one per slot, in shared memory)
// ----------------------------------------------------------------------------------------------
struct __align__(16) StepDesc {
  int32_t tile;
  int32_t link;
  uint32_t flags;
  uint32_t sent;                 // publication queue only: the step's frame went out
  uint32_t in_lo, in_hi;         // per in-ring r one byte: frames available << 6 | first slot
  uint32_t out_lo, out_hi;       // per out-ring r one byte: has room << 6 | next slot
};
constexpr uint32_t kDescFirst = 1;   // the tile's first step: the slot also holds the values
constexpr uint32_t kDescExit = 2;    // nothing more to do in this launch
constexpr uint32_t kDescRxAny = 4;   // at least one frame arrived for the tile
constexpr uint32_t kDescTxOk = 8;    // every out-ring of the link has room
constexpr uint32_t kDescRxLink = 16; // at least one frame arrived on this step's link
constexpr uint32_t kDescLast = 32;   // the tile's last step
constexpr uint32_t kDescNoValues = 128; // the step only receives: the values are not loaded, what arrived goes into them as a reduce-add
constexpr uint32_t kDescTxWant = 64; // the link may have something to hear: the tile changed here, or frames arrived on another link
constexpr uint32_t kFlagChanged = 1, kFlagNonsilent = 2, kFlagFailed = 4;  // what the compute warps report about a step

__device__ __forceinline__ uint32_t ctrl_byte(uint32_t lo, uint32_t hi, int r) { return ((r < 4 ? lo : hi) >> ((r & 3) * 8)) & 0xffu; }

struct SmemLayout {
  int slot_stride;  // values tile, mirror tile, payload
  int off_slots;    // [kGroups][kSlots][slot_stride]
  int off_desc;     // StepDesc[kGroups][kSlots]
  int off_pubq;     // StepDesc[kGroups][kPubQueue]
  int off_bar;      // uint64_t[kGroups][2 * kSlots + 1]: full, done, group sync
  int off_words;    // uint32_t[kGroups][16]: step flags per slot, armed steps, abort, publication counters
  int off_red;      // float[kGroups][2][8]: cross-warp partials for blocks of 2048 / 4096 elements
  int total;
};
__host__ __device__ inline SmemLayout smem_layout(int payload_bytes, int kGroups, int kSlots) {
  SmemLayout m;
  m.slot_stride = 2 * kTileBytes + ((payload_bytes + 127) & ~127);
  int off = 0;
  m.off_slots = off;
  off += kGroups * kSlots * m.slot_stride;
  m.off_desc = off;
  off += kGroups * kSlots * int(sizeof(StepDesc));
  m.off_pubq = off;
  off += kGroups * kPubQueue * int(sizeof(StepDesc));
  m.off_bar = off;
  off += kGroups * (2 * kSlots + 1) * 8;
  m.off_words = off;
  off += kGroups * 16 * 4;
  m.off_red = off;
  off += kGroups * 2 * 8 * 4;
  m.total = (off + 127) & ~127;
  return m;
}

// ----------------------------------------------------------------------------------------------
// per-thread arithmetic on 32 consecutive elements held as eight float4 pieces.  Register q holds the elements
// 4*(q^sw) .. +3 of the thread's 32 (sw = thread & 7, the shared-memory swizzle); a frame stores a thread's codes in
// the order of its registers, so the sender's and the receiver's thread of the same index agree without shuffling.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ int floor_log2_dev(float x) { return int((__float_as_uint(x) >> 23) & 0xff) - 127; }

// sign frames: step = 2^floor(log2(2/3 max|x|)), silent below the cut-off (block_code in ../core/codec.cpp)
__device__ __forceinline__ int block_code_sign(float xmax, uint32_t vmax_bits, int min_exp, int rel_bits) {
  const float scaled = __fmul_rn(xmax, 0.6666667f);
  if ((__float_as_uint(scaled) >> 23) == 0) return 0;
  int kx = floor_log2_dev(scaled);
  if (kx < min_exp) return 0;
  if ((vmax_bits >> 23) != 0) {
    int emax = int(vmax_bits >> 23) - 127;
    if (kx < emax - rel_bits) return 0;
  }
  if (kx < -126) return 0;
  if (kx > 127) kx = 127;
  return kx + 127;
}

// integer frames: the smallest step for which the largest residual still fits (block_code_int in ../core/codec.cpp)
template <int Q>
__device__ __forceinline__ int block_code_int_dev(float xmax, uint32_t vmax_bits, int min_exp, int rel_bits) {
  const uint32_t xb = __float_as_uint(xmax) & 0x7fffffffu;
  const int ef = int(xb >> 23);
  if (ef == 0 || ef == 255) return 0;
  const int ex = ef - 127;
  if (ex > 100) return 0;
  const uint32_t mant = xb & 0x7fffffu;
  int es = ex - (Q - 2);
  if (mant >= (1u << 23) - (1u << (24 - Q))) es += 1;
  es = max(es, min_exp);
  if ((vmax_bits >> 23) != 0) es = max(es, int((vmax_bits >> 23) & 0xffu) - 127 - rel_bits);
  es = max(es, -126);
  if (ex < es - 1 || (ex == es - 1 && mant == 0)) return 0;
  return es + 127;
}

template <int Q>
__device__ __forceinline__ int block_code_dev(float xmax, uint32_t vmax_bits, int min_exp, int rel_bits) {
  if constexpr (Q == 1) return block_code_sign(xmax, vmax_bits, min_exp, rel_bits);
  else return block_code_int_dev<Q>(xmax, vmax_bits, min_exp, rel_bits);
}

// the Q code words of thread t and the scale byte of its block, from a frame in a ring slot
template <int Q>
__device__ __forceinline__ void load_frame(const uint8_t* fp, int t, int tpb, uint32_t (&w)[Q], uint32_t& code) {
  const uint8_t* mine = fp + size_t(t) * (4 * Q);
  if (Q == 8) {
    const uint4 a = ld_cg_v4(mine), b = ld_cg_v4(mine + 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4 % Q] = b.x; w[5 % Q] = b.y; w[6 % Q] = b.z; w[7 % Q] = b.w;
  } else if (Q == 4) {
    const uint4 a = ld_cg_v4(mine);
    w[0] = a.x; w[1 % Q] = a.y; w[2 % Q] = a.z; w[3 % Q] = a.w;
  } else if (Q == 2) {
    const uint2 a = ld_cg_v2(mine);
    w[0] = a.x; w[1 % Q] = a.y;
  } else {
    w[0] = ld_cg_word(mine);
  }
  code = ld_cg_u8(fp + 4 * Q * kWordsPerTile + (t >> tpb));
}

// acc += the step the frame gives each of the 32 elements
template <int Q, bool MASKED>
__device__ __forceinline__ void add_frame(float4 (&acc)[8], const uint32_t (&w)[Q], uint32_t code, int sw, uint32_t vmask) {
  if (code == 0u || code == 255u) return;
  const float s = __uint_as_float(code << 23);
  if (Q == 1) {
    const uint32_t sb = code << 23;
#pragma unroll
    for (int q = 0; q < 8; q++) {
      const uint32_t wq = w[0] >> (4 * q);
      const float f0 = __uint_as_float(sb | ((wq << 31) & 0x80000000u)), f1 = __uint_as_float(sb | ((wq << 30) & 0x80000000u));
      const float f2 = __uint_as_float(sb | ((wq << 29) & 0x80000000u)), f3 = __uint_as_float(sb | ((wq << 28) & 0x80000000u));
      if (!MASKED) {
        acc[q].x = __fadd_rn(acc[q].x, f0); acc[q].y = __fadd_rn(acc[q].y, f1);
        acc[q].z = __fadd_rn(acc[q].z, f2); acc[q].w = __fadd_rn(acc[q].w, f3);
      } else {
        const uint32_t vq = vmask >> (4 * (q ^ sw));
        if (vq & 1u) acc[q].x = __fadd_rn(acc[q].x, f0);
        if (vq & 2u) acc[q].y = __fadd_rn(acc[q].y, f1);
        if (vq & 4u) acc[q].z = __fadd_rn(acc[q].z, f2);
        if (vq & 8u) acc[q].w = __fadd_rn(acc[q].w, f3);
      }
    }
  } else {
    // a code c stands for (c - 2^(Q-1)) steps; 2^23 + c as a float is 0x4B000000 | c
    const float big = 8388608.f + float(1 << (Q - 1));
    const float neg_ms = -__fmul_rn(big, s);
#pragma unroll
    for (int q = 0; q < 8; q++) {
      uint32_t z0, z1, z2, z3;
      if (Q == 8) {
        const uint32_t wq = w[q % Q];
        z0 = __byte_perm(wq, 0x4B000000u, 0x7650); z1 = __byte_perm(wq, 0x4B000000u, 0x7651);
        z2 = __byte_perm(wq, 0x4B000000u, 0x7652); z3 = __byte_perm(wq, 0x4B000000u, 0x7653);
      } else {
        constexpr uint32_t m = (1u << Q) - 1u;
        const uint32_t wq = w[(q * Q / 8) % Q] >> ((q * 4 * Q) & 31);  // 4*Q bits per register
        z0 = (wq & m) | 0x4B000000u; z1 = ((wq >> Q) & m) | 0x4B000000u;
        z2 = ((wq >> (2 * Q)) & m) | 0x4B000000u; z3 = ((wq >> (3 * Q)) & m) | 0x4B000000u;
      }
      acc[q].x = __fadd_rn(acc[q].x, __fmaf_rn(__uint_as_float(z0), s, neg_ms));
      acc[q].y = __fadd_rn(acc[q].y, __fmaf_rn(__uint_as_float(z1), s, neg_ms));
      acc[q].z = __fadd_rn(acc[q].z, __fmaf_rn(__uint_as_float(z2), s, neg_ms));
      acc[q].w = __fadd_rn(acc[q].w, __fmaf_rn(__uint_as_float(z3), s, neg_ms));
    }
  }
}

// the codes of v - k for a block with exponent code `code` (non-zero), and the mirror's step
template <int Q, bool MASKED>
__device__ __forceinline__ void quantise(const float4 (&v)[8], float4 (&k)[8], uint32_t code, uint32_t (&w)[Q], int sw, uint32_t vmask) {
  if (Q == 1) {
    const float sp = __uint_as_float(code << 23), sn = __uint_as_float((code << 23) | 0x80000000u);
    uint32_t word = 0;
#pragma unroll
    for (int q = 0; q < 8; q++) {
      const bool n0 = !(__fsub_rn(v[q].x, k[q].x) > 0.f), n1 = !(__fsub_rn(v[q].y, k[q].y) > 0.f);
      const bool n2 = !(__fsub_rn(v[q].z, k[q].z) > 0.f), n3 = !(__fsub_rn(v[q].w, k[q].w) > 0.f);
      uint32_t nib = (n0 ? 1u : 0u) | (n1 ? 2u : 0u) | (n2 ? 4u : 0u) | (n3 ? 8u : 0u);
      if (!MASKED) {
        k[q].x = __fadd_rn(k[q].x, n0 ? sn : sp); k[q].y = __fadd_rn(k[q].y, n1 ? sn : sp);
        k[q].z = __fadd_rn(k[q].z, n2 ? sn : sp); k[q].w = __fadd_rn(k[q].w, n3 ? sn : sp);
      } else {
        const uint32_t vq = (vmask >> (4 * (q ^ sw))) & 0xfu;
        nib &= vq;
        if (vq & 1u) k[q].x = __fadd_rn(k[q].x, n0 ? sn : sp);
        if (vq & 2u) k[q].y = __fadd_rn(k[q].y, n1 ? sn : sp);
        if (vq & 4u) k[q].z = __fadd_rn(k[q].z, n2 ? sn : sp);
        if (vq & 8u) k[q].w = __fadd_rn(k[q].w, n3 ? sn : sp);
      }
      word |= nib << (4 * q);
    }
    w[0] = word;
  } else {
    const float s = __uint_as_float(code << 23), inv = __uint_as_float((254u - code) << 23);
    const float big = 8388608.f + float(1 << (Q - 1));
    const float neg_ms = -__fmul_rn(big, s);
#pragma unroll
    for (int j = 0; j < Q; j++) w[j] = 0;
#pragma unroll
    for (int q = 0; q < 8; q++) {
      const float z0 = __fmaf_rn(__fsub_rn(v[q].x, k[q].x), inv, big), z1 = __fmaf_rn(__fsub_rn(v[q].y, k[q].y), inv, big);
      const float z2 = __fmaf_rn(__fsub_rn(v[q].z, k[q].z), inv, big), z3 = __fmaf_rn(__fsub_rn(v[q].w, k[q].w), inv, big);
      k[q].x = __fadd_rn(k[q].x, __fmaf_rn(z0, s, neg_ms)); k[q].y = __fadd_rn(k[q].y, __fmaf_rn(z1, s, neg_ms));
      k[q].z = __fadd_rn(k[q].z, __fmaf_rn(z2, s, neg_ms)); k[q].w = __fadd_rn(k[q].w, __fmaf_rn(z3, s, neg_ms));
      const uint32_t b0 = __float_as_uint(z0), b1 = __float_as_uint(z1), b2 = __float_as_uint(z2), b3 = __float_as_uint(z3);
      if (Q == 8) {
        w[q % Q] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
      } else {
        constexpr uint32_t m = (1u << Q) - 1u;
        const uint32_t four = (b0 & m) | ((b1 & m) << Q) | ((b2 & m) << (2 * Q)) | ((b3 & m) << (3 * Q));
        w[(q * Q / 8) % Q] |= four << ((q * 4 * Q) & 31);
      }
    }
  }
}

// largest |v - k| among the 32 elements
__device__ __forceinline__ float residual_maxabs(const float4 (&v)[8], const float4 (&k)[8]) {
  float m = 0.f;
#pragma unroll
  for (int q = 0; q < 8; q++) {
    m = fmaxf(fmaxf(m, fabsf(__fsub_rn(v[q].x, k[q].x))), fabsf(__fsub_rn(v[q].y, k[q].y)));
    m = fmaxf(fmaxf(m, fabsf(__fsub_rn(v[q].z, k[q].z))), fabsf(__fsub_rn(v[q].w, k[q].w)));
  }
  return m;
}
// bits of the largest |v| among the 32 elements
__device__ __forceinline__ uint32_t max_abs_bits(const float4 (&v)[8]) {
  float m = 0.f;
#pragma unroll
  for (int q = 0; q < 8; q++) m = fmaxf(fmaxf(fmaxf(m, fabsf(v[q].x)), fabsf(v[q].y)), fmaxf(fabsf(v[q].z), fabsf(v[q].w)));
  return __float_as_uint(m);
}

}  // namespace

int round_smem_bytes(int groups, int slots, int payload_bytes) { return smem_layout(payload_bytes, groups, slots).total; }

// ----------------------------------------------------------------------------------------------
// the kernel
// ----------------------------------------------------------------------------------------------
template <int Q, int kGroups, int kSlots>
__global__ void __launch_bounds__(kGroups * (kGroupThreads + 32) + 32, 1)
    round_kernel(const __grid_constant__ RoundParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const SmemLayout lay = smem_layout(p.payload_bytes, kGroups, kSlots);
  const int tid = threadIdx.x;
  const bool is_pub = tid >= kGroups * (kGroupThreads + 32);
  const bool is_io = !is_pub && tid >= kGroups * kGroupThreads;
  const int g = is_pub ? 0 : (is_io ? (tid - kGroups * kGroupThreads) >> 5 : tid >> 7);
  const int lane = tid & 31;
  uint8_t* slots = smem + lay.off_slots + size_t(g) * kSlots * lay.slot_stride;
  StepDesc* desc = reinterpret_cast<StepDesc*>(smem + lay.off_desc) + g * kSlots;
  StepDesc* pubq = reinterpret_cast<StepDesc*>(smem + lay.off_pubq) + g * kPubQueue;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bar) + g * (2 * kSlots + 1);
  uint64_t* done = full + kSlots;
  uint64_t* gsync = full + 2 * kSlots;
  uint32_t* words = reinterpret_cast<uint32_t*>(smem + lay.off_words) + g * 16;
  uint32_t* sflags = words;          // [kSlots]
  uint32_t* armed = words + 4;       // steps armed so far
  uint32_t* abort_flag = words + 5;
  uint32_t* pub_ready = words + 6;   // steps whose stores have completed (I/O warp -> publisher)
  uint32_t* pub_done = words + 7;    // steps published (publisher -> I/O warp)
  uint32_t* pub_exit = words + 8;    // the group's I/O warp has nothing more to publish
  uint32_t* yield_seen = reinterpret_cast<uint32_t*>(smem + lay.off_words) + 9;  // group 0's word: an update is waiting
  float* s_red = reinterpret_cast<float*>(smem + lay.off_red) + g * 16;

  if (tid == 0) {
    for (int i = 0; i < kGroups; i++) {
      uint64_t* b = reinterpret_cast<uint64_t*>(smem + lay.off_bar) + i * (2 * kSlots + 1);
      for (int s = 0; s < kSlots; s++) {
        mbar_init(b + s, 1);           // full: the I/O warp's arrive (+ the copies' bytes)
        mbar_init(b + kSlots + s, 4);  // done: one arrive per compute warp
      }
      mbar_init(b + 2 * kSlots, 4);    // group sync of the compute warps
      uint32_t* wd = reinterpret_cast<uint32_t*>(smem + lay.off_words) + i * 16;
      for (int j = 0; j < 16; j++) wd[j] = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncthreads();  // the only CTA-wide barrier: from here on the groups, and the two kinds of warp, run on their own

  const int L = p.n_links;
  const int pb = p.payload_bytes;
  const int tpb = p.log2_block - 5;  // log2(threads per block of the quantiser)
  const uint64_t limit_ns = p.wait_ns;
  uint64_t* const launch_words = p.status + (p.parity ? kDsLaunch1 : kDsLaunch0);

  if (is_pub) {
    // =========================================================================================
    // publisher warp: sequence flags and credits of the steps whose stores have completed, for every group of the
    // CTA.  Lane r serves out-ring r and in-ring r.
    // =========================================================================================
    uint32_t published[kGroups];
#pragma unroll
    for (int i = 0; i < kGroups; i++) published[i] = 0;
    const uint64_t t_start = globaltimer_ns();
    for (uint32_t it = 0;; it++) {
      ST_CRUMB(3, 20);
      // An update that is waiting for SMs: the I/O warps read this copy of the flag before they hand out a tile.
      if (p.yield_flag != nullptr && lane == 0 && ld_cg_u32(p.yield_flag) != 0u) st_shared_volatile(yield_seen, 1u);
      uint32_t ready[kGroups];
      bool any = false, all_exit = true;
#pragma unroll
      for (int i = 0; i < kGroups; i++) {
        uint32_t* wd = reinterpret_cast<uint32_t*>(smem + lay.off_words) + i * 16;
        // These words change under the warp's feet: lane 0 reads them and every lane takes lane 0's answer, so that
        // the warp decides as one.
        const uint32_t ex = __shfl_sync(0xffffffffu, ld_shared_volatile(wd + 8), 0);  // read before the counter: an exit
        all_exit &= ex != 0;                                                           // flag is set after the last hand-over
        ready[i] = __shfl_sync(0xffffffffu, ld_shared_volatile(wd + 6), 0);
        any |= ready[i] != published[i];
      }
      if (any) {
        ST_CRUMB(3, 21);
        __threadfence_block();
        __threadfence_system();  // the payloads are performed before the flags that announce them
        ST_CRUMB(3, 22);
#pragma unroll
        for (int i = 0; i < kGroups; i++) {
          const StepDesc* q = reinterpret_cast<const StepDesc*>(smem + lay.off_pubq) + i * kPubQueue;
          for (; published[i] != ready[i]; published[i]++) {
            const StepDesc e = q[published[i] & (kPubQueue - 1)];
            if (e.sent && lane < p.n_out && p.out[lane].link == e.link) {
              const uint32_t slot_no = ctrl_byte(e.out_lo, e.out_hi, lane) & 63u;
              const uint32_t seq = ld_cg_u32(p.out[lane].tx_seq + e.tile) + 1u;
              st_relaxed_sys(p.out[lane].flags_remote + size_t(slot_no) * p.n_tiles + e.tile, seq);
              st_cg_u32(p.out[lane].tx_seq + e.tile, seq);
            }
            if ((e.flags & kDescLast) && lane < p.n_in) {
              const uint32_t avail = ctrl_byte(e.in_lo, e.in_hi, lane) >> 6;
              if (avail) {
                const uint32_t seq = ld_cg_u32(p.in[lane].rx_seq + e.tile) + avail;
                st_cg_u32(p.in[lane].rx_seq + e.tile, seq);
                st_relaxed_sys(p.in[lane].credit_remote + e.tile, seq);
              }
            }
          }
          __syncwarp();
          __threadfence();  // the sequence counters are read by other warps once the hand-back below is seen
          if (lane == 0) st_shared_volatile(reinterpret_cast<uint32_t*>(smem + lay.off_words) + i * 16 + 7, published[i]);
        }
      } else {
        if (all_exit) break;
        __nanosleep(100);
        if ((it & 1023u) == 1023u && globaltimer_ns() - t_start > 4000ull * 1000 * 1000) break;  // the I/O warps are gone
      }
    }
    ST_CRUMB(3, 23);
    return;
  }

  if (!is_io) {
    // =========================================================================================
    // compute warps
    // =========================================================================================
    const int t = tid & 127;          // thread in group = 32-element chunk of the tile
    const int wig = (tid >> 5) & 3;   // warp in group
    const int sw = t & 7;             // XOR swizzle of this thread's eight 16-byte pieces
    const int64_t n = p.n;
    float res_max0 = 0.f, res_max1 = 0.f, res_max2 = 0.f;
    uint32_t gphase = 0;
    float4 v[8];
    uint32_t vmax_mine = 0;
#ifdef ST_ROUND_TIMING
    long long tm_wait = 0, tm_total0 = clock64(), tm_steps = 0, tm_a = 0, tm_b = 0, tm_c = 0, tm_d = 0, tm_e = 0, st_lap_ = 0;
#endif

    for (uint32_t c = 0;; c++) {
      const int s = int(c % kSlots);
      uint8_t* slot = slots + size_t(s) * lay.slot_stride;
      ST_CRUMB(4 + g, 30);
      ST_T0();
      // The step's descriptor first: it says which frames arrived, and their loads go out before the wait for the
      // tile, so that the two latencies overlap.
      const bool armed_ok = __all_sync(0xffffffffu, wait_armed(armed, c, abort_flag));  // the warp decides as one
      __threadfence_block();
      const StepDesc d = desc[s];
      if (armed_ok && (d.flags & kDescExit)) break;
      const int tile = d.tile, l = d.link;
      float4* slot_v = reinterpret_cast<float4*>(slot) + t * 8;
      float4* slot_k = reinterpret_cast<float4*>(slot + kTileBytes) + t * 8;
      const int64_t left = n - (int64_t(tile) * kTile + int64_t(t) * 32);  // elements of this thread's chunk that exist
      const bool full_chunk = left >= 32;
      const uint32_t vmask = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << int(left)) - 1u));
      const bool masked = (Q == 1) && !full_chunk;
      bool failed = false;

      // ---- frames, in ring order and sequence order.  `only_link` < 0 takes every ring.
      int it_r = -1, it_f = 0, it_avail = 0, it_only = -1;
      uint32_t it_ib = 0;
      auto first_frame = [&](int only_link) {
        it_r = -1; it_f = 0; it_avail = 0; it_only = only_link;
      };
      auto next_frame = [&]() -> const uint8_t* {
        while (true) {
          if (it_r >= 0 && it_f < it_avail) {
            const int slot_no = (int(it_ib & 63u) + it_f) & (p.ring_slots - 1);
            it_f++;
            return p.in[it_r].payload + (size_t(slot_no) * p.n_tiles + tile) * pb;
          }
          it_r++;
          if (it_r >= p.n_in) return nullptr;
          it_ib = ctrl_byte(d.in_lo, d.in_hi, it_r);
          it_avail = (it_only >= 0 && p.in[it_r].link != it_only) ? 0 : int(it_ib >> 6);
          it_f = 0;
        }
      };
      // Frames are fetched four at a time, so that four load latencies overlap, and applied in order.
      constexpr int kBatch = 4;
      uint32_t bw[kBatch][Q], bc[kBatch];
      int bn = 0;
      auto load_batch = [&]() {
        bn = 0;
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
          const uint8_t* fp = bn == i ? next_frame() : nullptr;
          if (fp) {
            load_frame<Q>(fp, t, tpb, bw[i], bc[i]);
            bn = i + 1;
          }
        }
      };
      // acc = the sum of the frames' steps; the first batch may have been fetched already
      auto decode_frames = [&](float4 (&acc)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        while (bn > 0) {
#pragma unroll
          for (int i = 0; i < kBatch; i++) {
            if (i < bn) {
              if (masked) add_frame<Q, true>(acc, bw[i], bc[i], sw, vmask); else add_frame<Q, false>(acc, bw[i], bc[i], sw, vmask);
            }
          }
          if (bn == kBatch) load_batch(); else bn = 0;
        }
      };

      const bool rx_first = armed_ok && (d.flags & kDescFirst) && (d.flags & kDescRxAny);
      if (rx_first) {
        first_frame(-1);
        load_batch();
      }
      ST_CRUMB(4 + g, 31);
      const bool step_ok = __all_sync(0xffffffffu, armed_ok && mbar_wait_bounded(full + s, (c / kSlots) & 1u, limit_ns));
      ST_CRUMB(4 + g, 32);
      if (wig == 0) ST_STAMP(c, 1);
      ST_ACC(tm_wait);
#ifdef ST_ROUND_TIMING
      tm_steps++;
#endif
      if (!step_ok) {
        // Nothing of this step is stored: the warp reports the failure and leaves; the I/O warp then stops the group.
        if (lane == 0) atomicOr(&sflags[s], kFlagFailed);
        __syncwarp();
        if (lane == 0) mbar_arrive(done + s);
        break;
      }

#ifdef ST_ROUND_TIMING
      st_lap_ = clock64();
#endif
      if (d.flags & kDescFirst) {
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = (d.flags & kDescNoValues) ? make_float4(0.f, 0.f, 0.f, 0.f) : slot_v[q ^ sw];
        if (rx_first) {
          float4 acc[8];
          decode_frames(acc);
#pragma unroll
          for (int q = 0; q < 8; q++) {
            v[q].x = __fadd_rn(v[q].x, acc[q].x); v[q].y = __fadd_rn(v[q].y, acc[q].y);
            v[q].z = __fadd_rn(v[q].z, acc[q].z); v[q].w = __fadd_rn(v[q].w, acc[q].w);
            slot_v[q ^ sw] = acc[q];  // leaves as a reduce-add into the values
          }
        }
        vmax_mine = max_abs_bits(v);
      }

      ST_LAP(tm_a);
      float4 k[8];
#pragma unroll
      for (int q = 0; q < 8; q++) k[q] = slot_k[q ^ sw];
      bool changed = false;
      if (d.flags & kDescRxLink) {
        float4 acc[8];
        if (L == 1) {
          // one link: what arrived for the values is what arrived on this link, and the slot still holds it
#pragma unroll
          for (int q = 0; q < 8; q++) acc[q] = slot_v[q ^ sw];
        } else {
          first_frame(l);
          load_batch();
          decode_frames(acc);
        }
#pragma unroll
        for (int q = 0; q < 8; q++) {
          k[q].x = __fadd_rn(k[q].x, acc[q].x); k[q].y = __fadd_rn(k[q].y, acc[q].y);
          k[q].z = __fadd_rn(k[q].z, acc[q].z); k[q].w = __fadd_rn(k[q].w, acc[q].w);
        }
        changed = true;
      }

      ST_LAP(tm_b);
      // ---- quantise values - mirror for link l
      const bool want = (d.flags & kDescTxWant) != 0;  // (a step that only receives says nothing back, whatever rounding left)
      float xm = residual_maxabs(v, k);
      if (!want) xm = 0.f;
      if (l == 0) res_max0 = fmaxf(res_max0, xm); else if (l == 1) res_max1 = fmaxf(res_max1, xm); else res_max2 = fmaxf(res_max2, xm);
      uint32_t vm = vmax_mine;
      // blocks larger than 32 elements: maximum over lanes (up to 1024), then over the group's warps
      for (int sft = 0; sft < tpb && sft < 5; sft++) {
        xm = fmaxf(xm, __shfl_xor_sync(0xffffffffu, xm, 1 << sft));
        vm = max(vm, __shfl_xor_sync(0xffffffffu, vm, 1 << sft));
      }
      if (tpb > 5) {
        float* red = s_red + (c & 1u) * 8;  // two buffers: a warp may be one step ahead of the slowest one
        if (lane == 0) {
          red[wig] = xm;
          red[4 + wig] = __uint_as_float(vm);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(gsync);
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(gsync, gphase, limit_ns))) failed = true;
        gphase ^= 1u;
        const float a0 = red[0], a1 = red[1], a2 = red[2], a3 = red[3];
        const uint32_t b0 = __float_as_uint(red[4]), b1 = __float_as_uint(red[5]);
        const uint32_t b2 = __float_as_uint(red[6]), b3 = __float_as_uint(red[7]);
        if (tpb == 6) {  // 2048: warps {0,1} and {2,3}
          xm = wig < 2 ? fmaxf(a0, a1) : fmaxf(a2, a3);
          vm = wig < 2 ? max(b0, b1) : max(b2, b3);
        } else {         // 4096: the whole tile
          xm = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
          vm = max(max(b0, b1), max(b2, b3));
        }
      }
      const int code = block_code_dev<Q>(xm, vm, p.min_exp, p.rel_bits);
      ST_LAP(tm_c);
      if ((d.flags & kDescTxOk) != 0) {
        uint8_t* pay = slot + 2 * kTileBytes;
        if (code) {
          uint32_t w[Q];
          if (masked) quantise<Q, true>(v, k, uint32_t(code), w, sw, vmask); else quantise<Q, false>(v, k, uint32_t(code), w, sw, vmask);
          changed = true;
          if (Q == 8) {
            reinterpret_cast<uint4*>(pay)[t * 2] = make_uint4(w[0], w[1 % Q], w[2 % Q], w[3 % Q]);
            reinterpret_cast<uint4*>(pay)[t * 2 + 1] = make_uint4(w[4 % Q], w[5 % Q], w[6 % Q], w[7 % Q]);
          } else if (Q == 4) {
            reinterpret_cast<uint4*>(pay)[t] = make_uint4(w[0], w[1 % Q], w[2 % Q], w[3 % Q]);
          } else if (Q == 2) {
            reinterpret_cast<uint2*>(pay)[t] = make_uint2(w[0], w[1 % Q]);
          } else {
            reinterpret_cast<uint32_t*>(pay)[t] = w[0];
          }
        }
        if ((t & ((1 << tpb) - 1)) == 0) pay[4 * Q * kWordsPerTile + (t >> tpb)] = uint8_t(code);
      }
      ST_LAP(tm_d);
      if (changed) {
#pragma unroll
        for (int q = 0; q < 8; q++) slot_k[q ^ sw] = k[q];
      }
      fence_async_smem();  // what this thread wrote into the slot is about to be read by bulk stores
      {
        const uint32_t mine = (changed ? kFlagChanged : 0u) | (code ? kFlagNonsilent : 0u) | (failed ? kFlagFailed : 0u);
        const uint32_t warp_bits = __reduce_or_sync(0xffffffffu, mine);
        if (lane == 0 && warp_bits) atomicOr(&sflags[s], warp_bits);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(done + s);
      if (wig == 0) ST_STAMP(c, 2);
      ST_LAP(tm_e);
      if (failed) break;
    }

#ifdef ST_ROUND_TIMING
    if (blockIdx.x == 0 && tid == 0)
      printf("compute: total %lld cycles, waiting for steps %lld, steps %lld; values+decode %lld, mirror+rx %lld, stats %lld, quantise %lld, store+arrive %lld\n",
             clock64() - tm_total0, tm_wait, tm_steps, tm_a, tm_b, tm_c, tm_d, tm_e);
#endif
    ST_CRUMB(4 + g, 33);
    // ---- statistics: the largest outstanding residual per link
    {
      float a0 = res_max0, a1 = res_max1, a2 = res_max2;
      for (int o = 16; o > 0; o >>= 1) {
        a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, o));
        a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, o));
        a2 = fmaxf(a2, __shfl_xor_sync(0xffffffffu, a2, o));
      }
      if (lane == 0) {  // non-negative floats order like their bit patterns
        unsigned long long* rm = reinterpret_cast<unsigned long long*>(launch_words + kDlResMax);
        if (a0 != 0.f) atomicMax(rm + 0, (unsigned long long)__float_as_uint(a0));
        if (a1 != 0.f) atomicMax(rm + 1, (unsigned long long)__float_as_uint(a1));
        if (a2 != 0.f) atomicMax(rm + 2, (unsigned long long)__float_as_uint(a2));
      }
    }
    return;
  }

  // ===========================================================================================
  // I/O warp.  All 32 lanes run the same control flow; lane 0 issues copies, stores and flags.
  // ===========================================================================================
  // The group's tiles: a run of `chunk` consecutive tiles, or (chunk == 0) every gstride-th tile of the tensor.
  // (of the launch's window of the tensor, tiles tile_begin .. tile_begin + tile_count - 1)
  const int gidx = int(blockIdx.x) * kGroups + g;
  const int gid0 = p.chunk > 0 ? gidx * p.chunk : gidx;
  const int gstride = p.chunk > 0 ? 1 : int(gridDim.x) * kGroups;
  const int my_count = p.chunk > 0 ? max(0, min(p.chunk, p.tile_count - gid0))
                                   : (p.tile_count > gid0 ? (p.tile_count - gid0 + gstride - 1) / gstride : 0);
  const int gid = p.tile_begin + gid0;
  const uint32_t smask = uint32_t(p.ring_slots) - 1u;
  uint32_t issued = 0, retired = 0;
  unsigned long long n_done = 0, n_tx = 0, n_rx = 0, n_blocked = 0, n_pending = 0, n_sweeps = 0;
  bool aborted = false, tile_pending = false, yielded = false;
#ifdef ST_ROUND_TIMING
  long long tm_done = 0, tm_read = 0, tm_pubwait = 0, tm_pub = 0, tm_scout = 0, tm_issue = 0, tm_store = 0, tm_pf = 0, tm_io0 = clock64();
#endif

  if (p.zero_other && blockIdx.x == 0 && g == 0 && lane == 0) {
    uint64_t* other = p.status + (p.parity ? kDsLaunch0 : kDsLaunch1);  // the next cycle's half
    for (int i = 0; i < 8; i++) other[i] = 0;
  }

  // Steps whose stores have completed are handed to the publisher warp; `pushed` counts the steps queued so far.
  uint32_t pushed = 0, handed = 0;
  auto hand_over = [&](uint32_t upto) {
    if (lane == 0 && upto != handed) {
      __threadfence_block();
      st_shared_volatile(pub_ready, upto);
    }
    handed = upto;
  };
  // bounded wait until the publisher has published `upto` steps
  auto wait_published = [&](uint32_t upto) -> bool {
    const uint64_t t0 = globaltimer_ns();
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 26); it++) {
      if (int32_t(ld_shared_volatile(pub_done) - upto) >= 0) {
        ok = true;
        break;
      }
      if ((it & 15) == 15 && globaltimer_ns() - t0 > 2 * limit_ns + 2000000ull) break;
      __nanosleep(50);
    }
    return __all_sync(0xffffffffu, ok);  // the warp decides as one
  };

  // a finished step: its stores go out and its slot becomes free
  auto retire = [&](uint32_t c) -> bool {
    const int s = int(c % kSlots);
    bool ok;
    {
      ST_T0();
      ST_CRUMB(g, 4);
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(done + s, (c / kSlots) & 1u, 2 * limit_ns));
      ST_ACC(tm_done);
    }
    ST_STAMP(c, 3);
    const uint32_t f = ok ? __shfl_sync(0xffffffffu, ld_shared_volatile(sflags + s), 0) : kFlagFailed;
    if (f & kFlagFailed) return false;
    if (pushed - __shfl_sync(0xffffffffu, ld_shared_volatile(pub_done), 0) >= uint32_t(kPubQueue)) {  // (the publisher has fallen behind: its fence takes tens of microseconds under load)
      bulk_wait_all();
      __syncwarp();
      hand_over(pushed);
      if (!wait_published(pushed)) return false;
    }
    ST_T0();
    {
      // the step's stores, one per lane, issued by as few instructions as possible: lane 0 the reduce-add of what was
      // received into the values; lane 1 the stepped mirror, lanes 2.. the frame into the ring of out-ring lane-2.
      // Every lane that issued commits and later waits for its own bulk group.
      const StepDesc d = desc[s];
      uint8_t* slot = slots + size_t(s) * lay.slot_stride;
      const bool sent = (d.flags & kDescTxOk) != 0 && (f & kFlagNonsilent) != 0;
      if (lane == 0 && (d.flags & kDescFirst) && (d.flags & kDescRxAny))
        bulk_reduce_add_f32(p.values + size_t(d.tile) * kTile, slot, kTileBytes);
      {
        void* dst = nullptr;
        const uint8_t* src = nullptr;
        uint32_t bytes = 0;
        if (lane == 1) {
          if (f & kFlagChanged) {
            dst = p.mirror[d.link] + size_t(d.tile) * kTile;
            src = slot + kTileBytes;
            bytes = kTileBytes;
          }
        } else if (lane >= 2 && lane - 2 < p.n_out && sent && p.out[lane - 2].link == d.link) {
          const uint32_t slot_no = ctrl_byte(d.out_lo, d.out_hi, lane - 2) & 63u;
          dst = p.out[lane - 2].payload_remote + (size_t(slot_no) * p.n_tiles + d.tile) * pb;
          src = slot + 2 * kTileBytes;
          bytes = uint32_t(pb);
        }
        if (bytes) bulk_s2g(dst, src, bytes);
      }
      bulk_commit();
    }
    if (lane == 0) {
      const StepDesc d = desc[s];
      const bool sent = (d.flags & kDescTxOk) != 0 && (f & kFlagNonsilent) != 0;
      if (sent)
        for (int r = 0; r < p.n_out; r++) n_tx += p.out[r].link == d.link ? 1 : 0;
      StepDesc e = d;
      e.sent = sent ? 1u : 0u;
      pubq[pushed & (kPubQueue - 1)] = e;
      if (f & kFlagNonsilent) {
        tile_pending = true;  // more may be left to say (or nothing could be said at all)
        if (!sent && p.do_tx) n_blocked++;
      }
      if (d.flags & kDescLast) {
        if (tile_pending) {
          st_cg_u32(p.tile_state + d.tile, 1u);
          n_pending++;
        }
        tile_pending = false;
        n_done++;
        for (int r = 0; r < p.n_in; r++) n_rx += ctrl_byte(d.in_lo, d.in_hi, r) >> 6;
      }
    }
    {
      ST_T0();
      ST_CRUMB(g, 5);
      bulk_wait_read_all();  // every lane for its own stores: the slot may be refilled
      ST_ACC(tm_read);
    }
    pushed++;
    __syncwarp();
    ST_STAMP(c, 4);
    ST_ACC(tm_store);
    return true;
  };

  ST_CRUMB(g, 1);
  for (int sweep = 0; sweep < p.sweeps && !aborted && !yielded && my_count > 0; sweep++) {
    const unsigned long long done_before = n_done;
    int scan_pos = 0;
    uint32_t pend = 0;                 // lanes whose scouted tile still has to be handed out
    int sc_tile = 0;                   // what this lane found for its tile
    uint32_t sc_in_lo = 0, sc_in_hi = 0, sc_out_lo = 0, sc_out_hi = 0, sc_dirty = 0;
    int cur_tile = -1, cur_a = 0;      // the tile whose steps are being handed out
    uint32_t cur_in_lo = 0, cur_in_hi = 0, cur_out_lo = 0, cur_out_hi = 0, cur_dirty = 0;
    bool exhausted = my_count == 0;

    while (true) {
      ST_CRUMB(g, 2);
      if (!exhausted && issued - retired < uint32_t(kSlots)) {
        if (cur_tile < 0 && __shfl_sync(0xffffffffu, ld_shared_volatile(yield_seen), 0) != 0u) {
          // An update is waiting for the SMs this kernel holds: hand out nothing more.  Tiles that were looked at but
          // not handed out get their change marks back, everything else is untouched.
          if (((pend >> lane) & 1u) && sc_dirty) st_cg_u32(p.tile_state + sc_tile, 1u);
          pend = 0;
          exhausted = true;
          yielded = true;
          continue;
        }
        if (cur_tile < 0) {
          if (pend == 0) {
            if (scan_pos >= my_count) {
              exhausted = true;
              continue;
            }
            // ---- look at 32 tiles at once, one per lane
            ST_T0();
            const int j = scan_pos + lane;
            const bool valid = j < my_count;
            sc_tile = gid + j * gstride;
            sc_in_lo = sc_in_hi = sc_out_lo = sc_out_hi = sc_dirty = 0;
            bool work = false;
            if (valid) {
              uint32_t dirty = ld_cg_u32(p.tile_state + sc_tile);
              bool any = false;
              if (p.do_rx) {
                for (int r = 0; r < p.n_in; r++) {
                  const uint32_t e = ld_cg_u32(p.in[r].rx_seq + sc_tile);
                  uint32_t avail = 0;
                  while (avail < uint32_t(kRxMax)) {
                    const uint32_t fl = ld_acquire_sys(p.in[r].flags + size_t((e + avail) & smask) * p.n_tiles + sc_tile);
                    if (fl != e + avail + 1u) break;
                    avail++;
                  }
                  const uint32_t byte = (avail << 6) | (e & smask);
                  if (r < 4) sc_in_lo |= byte << (r * 8); else sc_in_hi |= byte << ((r - 4) * 8);
                  any |= avail != 0;
                }
              }
              if (p.do_tx) {
                for (int r = 0; r < p.n_out; r++) {
                  const uint32_t tx = ld_cg_u32(p.out[r].tx_seq + sc_tile);
                  const uint32_t cr = ld_acquire_sys(p.out[r].credit + sc_tile);
                  const uint32_t room = (tx - cr) < uint32_t(p.ring_slots) ? 1u : 0u;
                  const uint32_t byte = (room << 6) | (tx & smask);
                  if (r < 4) sc_out_lo |= byte << (r * 8); else sc_out_hi |= byte << ((r - 4) * 8);
                }
              }
              // The change mark is cleared before the tile's values are read (the copy is issued after this
              // exchange has returned), and whoever changes the values sets it after the change: a change
              // that this visit does not see leaves its mark for the next one.
              if (dirty) dirty = atomicExch(p.tile_state + sc_tile, 0u);
              sc_dirty = dirty;
              work = dirty != 0 || any;
            }
            pend = __ballot_sync(0xffffffffu, work);
            scan_pos += 32;
            ST_ACC(tm_scout);
            continue;
          }
          const int src = __ffs(pend) - 1;
          pend &= pend - 1;
          cur_tile = __shfl_sync(0xffffffffu, sc_tile, src);
          cur_in_lo = __shfl_sync(0xffffffffu, sc_in_lo, src);
          cur_in_hi = __shfl_sync(0xffffffffu, sc_in_hi, src);
          cur_out_lo = __shfl_sync(0xffffffffu, sc_out_lo, src);
          cur_out_hi = __shfl_sync(0xffffffffu, sc_out_hi, src);
          cur_dirty = __shfl_sync(0xffffffffu, sc_dirty, src);
          cur_a = 0;
        }
        // ---- hand out step (cur_tile, link cur_a)
        ST_T0();
        __syncwarp();
        ST_ACC(tm_pf);
        // A tile of a one-link replica that carries no mark is here only to receive: nothing is said on the link, so
        // the values themselves are not needed (a third of the step's loads).
        const bool no_values = L == 1 && cur_dirty == 0;
        if (lane == 0) {
          const int s = int(issued % kSlots);
          uint8_t* slot = slots + size_t(s) * lay.slot_stride;
          const int l = cur_a;
          bool tx_any = false, tx_room = true, rx_link = false;
          for (int r = 0; r < p.n_out; r++) {
            if (p.out[r].link != l) continue;
            tx_any = true;
            tx_room &= (ctrl_byte(cur_out_lo, cur_out_hi, r) >> 6) != 0;
          }
          // A frame that arrived on link l changes the values and l's mirror alike: it leaves nothing to say on l, and
          // what rounding makes of it (or a cut-off that moved with the values) is not worth a frame back.  The link
          // gets a frame when the tile changed here (its mark) or when another link brought something to pass on.
          bool rx_other = false;
          for (int r = 0; r < p.n_in; r++) {
            if ((ctrl_byte(cur_in_lo, cur_in_hi, r) >> 6) == 0) continue;
            if (p.in[r].link == l) rx_link = true; else rx_other = true;
          }
          const bool tx_want = cur_dirty != 0 || rx_other;
          const bool rx_any = ((cur_in_lo | cur_in_hi) & 0xc0c0c0c0u) != 0;
          StepDesc d;
          d.tile = cur_tile;
          d.link = l;
          d.flags = (cur_a == 0 ? kDescFirst : 0u) | (rx_any ? kDescRxAny : 0u) | (tx_any && tx_room && tx_want && p.do_tx ? kDescTxOk : 0u) |
                    (rx_link ? kDescRxLink : 0u) | (tx_want ? kDescTxWant : 0u) | (no_values ? kDescNoValues : 0u) | (cur_a == L - 1 ? kDescLast : 0u);
          d.sent = 0;
          d.in_lo = cur_in_lo; d.in_hi = cur_in_hi; d.out_lo = cur_out_lo; d.out_hi = cur_out_hi;
          desc[s] = d;
          sflags[s] = 0;
          __threadfence_block();
          st_shared_volatile(armed, issued + 1u);  // the compute warps may read the descriptor from here on
          uint32_t bytes = (cur_a == 0 && !no_values ? 2u : 1u) * uint32_t(kTileBytes);
          if (cur_tile == p.stall_tile) bytes += 16;  // test hook: this barrier never completes
          mbar_expect_tx(full + s, bytes);
        }
        __syncwarp();
        {
          // the step's copies, one per lane, issued by one instruction: lane 0 the link's mirror, lane 1 the values
          const int s = int(issued % kSlots);
          uint8_t* slot = slots + size_t(s) * lay.slot_stride;
          if (lane == 0 || (lane == 1 && cur_a == 0 && !no_values)) {
            const float* src = (lane == 0 ? p.mirror[cur_a] : p.values) + size_t(cur_tile) * kTile;
            bulk_g2s(slot + (lane == 0 ? kTileBytes : 0), src, kTileBytes, full + s);
          }
        }
        ST_STAMP(issued, 0);
        issued++;
        cur_a++;
        if (cur_a == L) cur_tile = -1;
        __syncwarp();
        ST_ACC(tm_issue);
        continue;
      }
      // Nothing can be handed out right now: the steps whose stores have had time to land (all but the two most
      // recent) go to the publisher warp.
      if (pushed - handed > 2) {
        ST_T0();
        ST_CRUMB(g, 6);
        bulk_wait_all_but_2();  // every lane for its own stores
        hand_over(pushed - 2);
        ST_ACC(tm_pubwait);
      }
      if (retired < issued) {
        if (!retire(retired)) {
          aborted = true;
          break;
        }
        retired++;
        continue;
      }
      break;  // every tile looked at, every step retired
    }
    if (aborted) break;
    // ---- end of the sweep: every store has landed and is published before the tiles are looked at again
    ST_CRUMB(g, 7);
    bulk_wait_all();
    __syncwarp();
    hand_over(pushed);
    {
      ST_T0();
      ST_CRUMB(g, 8);
      if (!wait_published(pushed)) aborted = true;  // the next sweep reads the counters the publisher advances
      ST_ACC(tm_pub);
    }
    ST_CRUMB(g, 9);
    __syncwarp();
    if (aborted) break;
    n_sweeps++;
    if (n_done == done_before && sweep + 1 < p.sweeps) __nanosleep(1000);
  }

  if (aborted) {
    // Stop the group.  The compute warps leave on the abort flag (or on the exit descriptor); copies that are still
    // on their way get a bounded chance to land before the CTA's shared memory is released; what was stored is
    // published; every tile of the group is marked for another visit.
    if (lane == 0) st_shared_volatile(abort_flag, 1u);
    __syncwarp();
    for (uint32_t c = retired; c < issued; c++)
      (void)__all_sync(0xffffffffu, mbar_wait_bounded(full + int(c % kSlots), (c / kSlots) & 1u, limit_ns));
    bulk_wait_all();
    __syncwarp();
    hand_over(pushed);
    (void)wait_published(pushed);
    for (int j = lane; j < my_count; j += 32) st_cg_u32(p.tile_state + gid + j * gstride, 1u);
    if (lane == 0) {
      atomicOr(reinterpret_cast<unsigned long long*>(p.status + kDsErrors), (unsigned long long)kErrBarrierTimeout);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsWaitTimeouts), 1ull);
    }
  }
#ifdef ST_ROUND_TIMING
  if (blockIdx.x == 0 && g == 0 && lane == 0)
    printf("io: total %lld cycles, wait done %lld, wait read %lld, wait stores %lld, fence+publish %lld, scout %lld, prefetch %lld, issue(incl prefetch) %lld, retire(incl read wait) %lld, steps %u\n",
           clock64() - tm_io0, tm_done, tm_read, tm_pubwait, tm_pub, tm_scout, tm_pf, tm_issue, tm_store, issued);
#endif
  if (lane == 0) {
    // tell the compute warps that the launch is over (the slot of step `issued` is free: all earlier steps are retired
    // or abandoned)
    const int s = int(issued % kSlots);
    StepDesc d;
    d.tile = 0; d.link = 0; d.flags = kDescExit; d.sent = 0;
    d.in_lo = d.in_hi = d.out_lo = d.out_hi = 0;
    if (!aborted) {  // (after an abort the compute warps leave on the abort flag)
      desc[s] = d;
      __threadfence_block();
      st_shared_volatile(armed, issued + 1u);
      mbar_arrive(full + s);
    }
    st_shared_volatile(pub_exit, 1u);
    ST_CRUMB(g, 10);
    if (yielded) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsYields), 1ull);
    if (n_done) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsTilesProcessed), n_done);
    if (n_tx) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsFramesSent), n_tx);
    if (n_rx) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsFramesRecv), n_rx);
    if (n_blocked) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsBlockedNoCredit), n_blocked);
    if (n_done) atomicAdd(reinterpret_cast<unsigned long long*>(launch_words + kDlWork), n_done);
    if (n_pending) atomicAdd(reinterpret_cast<unsigned long long*>(launch_words + kDlPending), n_pending);
    if (blockIdx.x == 0 && g == 0) {
      const unsigned long long r = atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kDsSweeps), n_sweeps);
      uint64_t* rec = p.status + kDsTrace + (uint64_t(p.round) % kTraceEntries) * kTraceWords;  // trace ring, read by stats()
      rec[0] = globaltimer_ns();
      rec[1] = uint64_t(p.round);
      rec[2] = n_done;
      rec[3] = p.status[kDsFramesSent];
      (void)r;
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Taking frames back.  When a neighbour is lost, the frames it never acknowledged (sequence numbers from its last
// credit up to what was sent) are still in its ring, which stays mapped here; their steps come off the mirror again,
// so that what they said counts as not yet told (the TCP edges do the same with a frame whose write fails).
// One CTA per tile, thread t its 32 elements, the same element order as the round kernel.
// ----------------------------------------------------------------------------------------------
template <int Q>
__global__ void __launch_bounds__(kGroupThreads) unsend_kernel(float* __restrict__ mirror, const uint8_t* __restrict__ payload,
                                                               uint32_t* __restrict__ tx_seq, const uint32_t* __restrict__ credit,
                                                               int n_tiles, int ring_slots, int pb, int log2_block, int64_t n,
                                                               unsigned long long* __restrict__ taken_back) {
  const int tile = blockIdx.x, t = threadIdx.x, sw = t & 7, tpb = log2_block - 5;
  const uint32_t c = ld_acquire_sys(credit + tile), tx = ld_cg_u32(tx_seq + tile);
  const uint32_t count = tx - c;
  if (count == 0 || count > uint32_t(ring_slots)) return;
  const int64_t left = n - (int64_t(tile) * kTile + int64_t(t) * 32);
  const uint32_t vmask = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << int(left)) - 1u));
  const bool masked = (Q == 1) && left < 32;
  float4 acc[8];
#pragma unroll
  for (int q = 0; q < 8; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t f = 0; f < count; f++) {
    const uint8_t* fp = payload + (size_t((c + f) & uint32_t(ring_slots - 1)) * n_tiles + tile) * pb;
    uint32_t w[Q], code;
    load_frame<Q>(fp, t, tpb, w, code);
    if (masked) add_frame<Q, true>(acc, w, code, sw, vmask); else add_frame<Q, false>(acc, w, code, sw, vmask);
  }
  float4* k4 = reinterpret_cast<float4*>(mirror + size_t(tile) * kTile) + t * 8;
#pragma unroll
  for (int q = 0; q < 8; q++) {
    float4 k = k4[q ^ sw];
    k.x = __fsub_rn(k.x, acc[q].x); k.y = __fsub_rn(k.y, acc[q].y); k.z = __fsub_rn(k.z, acc[q].z); k.w = __fsub_rn(k.w, acc[q].w);
    k4[q ^ sw] = k;
  }
  __syncthreads();
  if (t == 0) {
    st_cg_u32(tx_seq + tile, c);
    atomicAdd(taken_back, (unsigned long long)count);
  }
}

int launch_unsend(float* mirror, const uint8_t* payload_remote, uint32_t* tx_seq, const uint32_t* credit, int n_tiles, int ring_slots,
                  int payload_bytes, int log2_block, int bits, int64_t n, uint64_t* taken_back, void* stream_v) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_v);
  unsigned long long* tb = reinterpret_cast<unsigned long long*>(taken_back);
  switch (bits) {
    case 1: unsend_kernel<1><<<n_tiles, kGroupThreads, 0, s>>>(mirror, payload_remote, tx_seq, credit, n_tiles, ring_slots, payload_bytes, log2_block, n, tb); break;
    case 2: unsend_kernel<2><<<n_tiles, kGroupThreads, 0, s>>>(mirror, payload_remote, tx_seq, credit, n_tiles, ring_slots, payload_bytes, log2_block, n, tb); break;
    case 4: unsend_kernel<4><<<n_tiles, kGroupThreads, 0, s>>>(mirror, payload_remote, tx_seq, credit, n_tiles, ring_slots, payload_bytes, log2_block, n, tb); break;
    case 8: unsend_kernel<8><<<n_tiles, kGroupThreads, 0, s>>>(mirror, payload_remote, tx_seq, credit, n_tiles, ring_slots, payload_bytes, log2_block, n, tb); break;
    default: return int(cudaErrorInvalidValue);
  }
  return int(cudaGetLastError());
}

// ----------------------------------------------------------------------------------------------
// launcher
// ----------------------------------------------------------------------------------------------
template <int Q, int G, int S>
static int launch_round_t(const RoundParams& p, int ctas, cudaStream_t stream) {
  const int smem = smem_layout(p.payload_bytes, G, S).total;
  static int configured_for = -1;  // per instantiation
  if (configured_for < smem) {
    cudaError_t e = cudaFuncSetAttribute(round_kernel<Q, G, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    configured_for = smem;
  }
  round_kernel<Q, G, S><<<ctas, G * (kGroupThreads + 32) + 32, smem, stream>>>(p);
  return int(cudaGetLastError());
}

template <int Q>
static int launch_round_q(const RoundParams& p, int shape, int ctas, cudaStream_t stream) {
  switch (shape) {
    case 0: return launch_round_t<Q, 3, 2>(p, ctas, stream);
    case 1: return launch_round_t<Q, 2, 3>(p, ctas, stream);
    default: return int(cudaErrorInvalidValue);
  }
}

int round_shape_groups(int shape) { return shape == 0 ? 3 : 2; }

int launch_round(const RoundParams& p, int shape, int ctas, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.n_links < 1 || p.n_links > kMaxLinks || p.sweeps < 1 || ctas < 1) return int(cudaErrorInvalidValue);
  if (p.ring_slots < 2 || p.ring_slots > 64 || (p.ring_slots & (p.ring_slots - 1))) return int(cudaErrorInvalidValue);
  switch (p.bits) {
    case 1: return launch_round_q<1>(p, shape, ctas, stream);
    case 2: return launch_round_q<2>(p, shape, ctas, stream);
    case 4: return launch_round_q<4>(p, shape, ctas, stream);
    case 8: return launch_round_q<8>(p, shape, ctas, stream);
    default: return int(cudaErrorInvalidValue);
  }
}

}  // namespace st
