// Sync-round kernels for sm_100a: round_begin, round_main and round_publish (see round.h for the protocol).
//
// round_main is the fused hot path.  A CTA is three independent groups of 128 threads; a group works
// through its share of the listed tiles, one 16 KB array-tile (values, then each link's mirror) at a time:
//   1. array-tiles are staged into shared memory with 1-D TMA bulk copies (cp.async.bulk, completion on an
//      mbarrier, a three-slot ring per group so the next copy is in flight while this one is computed;
//      every source is this GPU's own memory);
//   2. a thread owns 32 consecutive elements (read with an XOR swizzle, so no bank conflicts) and keeps its
//      values in registers for the whole tile; in a link's step it decodes the frames that arrived on that
//      link (sign bit + per-block power-of-two scale) once and adds them to the values and to the link's
//      mirror                                             (reference src/sharedtensor.c:106-111, 124-127);
//   3. per link it forms the residual values - mirror, the block's sum of squares, the exponent code from
//      the float's exponent bits, its 32 sign bits as one word, and steps the mirror by -/+ 2^k
//                                                         (reference 156-174);
//   4. changed mirror tiles and the tile's values go back to global memory with TMA bulk stores, and the packed words + scale bytes go straight into the neighbours' ring slots with
//      TMA bulk stores over NVLink
//      (reference 176-177: two socket writes).
// Nothing in here waits for another GPU.  The only waits are on this CTA's own TMA copies, and they are
// bounded: on a timeout the group records an error in the status block and leaves.
//
// Arithmetic is written with explicit round-to-nearest operations; block statistics are maxima (order does not
// matter), so words, scales and mirrors are bit-identical to the host codec (../core/codec.cpp).
#include <cuda_runtime.h>

#include <cstdint>

#include "round.h"

namespace st {

namespace {


constexpr int kGroupThreads = 128;  // one thread per 32 consecutive elements of a tile
__host__ __device__ constexpr int slots_for(int) { return 3; }  // array-tile slots per group
constexpr int kTileBytes = kTile * 4;

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
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait on one of this CTA's own copy barriers.  20 ms is three orders of magnitude above the
// time a stage takes; running into it means the copy was mis-issued, and the caller bails out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < (1u << 24); it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63) == 63 && globaltimer_ns() - t0 > 20ull * 1000 * 1000) return false;
  }
  return false;
}

__device__ __forceinline__ int floor_log2_dev(float x) { return int((__float_as_uint(x) >> 23) & 0xff) - 127; }

// exponent code of a block from its largest |residual| and the bits of its largest |value| (see block_code in
// ../core/codec.cpp: step = 2^floor(log2(2/3 max|x|)), silent below 2^(emax - rel_bits))
__device__ __forceinline__ int block_code_dev(float xmax, uint32_t vmax_bits, int min_exp, int rel_bits) {
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

}  // namespace

// ----------------------------------------------------------------------------------------------
// round_publish / round_begin: one thread per tile
// ----------------------------------------------------------------------------------------------
// After round_main: tell the neighbours what happened.  Credits for the frames this replica consumed
// go to their senders, sequence flags for the frames it wrote go to their receivers.  round_main has
// completed (stream order), so its peer stores are performed; one system-scope fence per publishing
// thread orders them before the flag stores that follow it.
__global__ void __launch_bounds__(256) round_publish_kernel(const __grid_constant__ RoundParams p) {
  const int tile = blockIdx.x * blockDim.x + threadIdx.x;
  if (tile >= p.n_tiles) return;
  uint8_t* cptr = p.ctrl + size_t(tile) * 16;
  const uint4 prev = *reinterpret_cast<const uint4*>(cptr);
  const uint8_t* pc = reinterpret_cast<const uint8_t*>(&prev);
  const uint2 sentw = *reinterpret_cast<const uint2*>(p.sent + size_t(tile) * 8);
  const uint8_t* ps = reinterpret_cast<const uint8_t*>(&sentw);
  if ((prev.x | prev.y) == 0u && (sentw.x | sentw.y) == 0u) return;  // nothing consumed, nothing sent
  __threadfence_system();
  for (int r = 0; r < p.n_in; r++) {
    int avail = pc[r] >> 6;
    if (avail) {
      uint32_t seq = p.in[r].rx_seq[tile] + uint32_t(avail);
      p.in[r].rx_seq[tile] = seq;
      st_relaxed_sys(p.in[r].credit_remote + tile, seq);
    }
  }
  for (int r = 0; r < p.n_out; r++) {
    const int frames = ps[r];  // frames written for this ring, in consecutive slots
    if (frames) {
      uint32_t seq = p.out[r].tx_seq[tile];
      const int slot0 = pc[8 + r] & 63;
      for (int f = 0; f < frames; f++) {
        seq++;
        st_relaxed_sys(p.out[r].flags_remote + size_t((slot0 + f) % p.ring_slots) * p.n_tiles + tile, seq);
      }
      p.out[r].tx_seq[tile] = seq;
    }
  }
  *reinterpret_cast<uint4*>(cptr) = make_uint4(0u, 0u, 0u, 0u);
  *reinterpret_cast<uint2*>(p.sent + size_t(tile) * 8) = make_uint2(0u, 0u);
}

// Before round_main: look at every tile's rings once (frames that arrived, ring space) and list the
// tiles that have something to do.
__global__ void __launch_bounds__(256) round_begin_kernel(const __grid_constant__ RoundParams p) {
  const int tile = blockIdx.x * blockDim.x + threadIdx.x;
  const int par = p.round & 1;
  if (tile == 0) {
    p.work_count[par ^ 1] = 0;  // the next round appends to the other counter
    p.status[kStPendingTiles] = 0;
    p.status[kStResidualMax0] = 0;
    p.status[kStResidualMax1] = 0;
    p.status[kStResidualMax2] = 0;
  }
  if (tile >= p.n_tiles) return;
  uint4 cur = make_uint4(0u, 0u, 0u, 0u);
  uint8_t* cc = reinterpret_cast<uint8_t*>(&cur);
  bool work = p.tile_state[tile] != 0;
  const uint32_t S = uint32_t(p.ring_slots);
  if (p.do_rx) {
    for (int r = 0; r < p.n_in; r++) {
      uint32_t e = p.in[r].rx_seq[tile];
      int avail = 0;
      while (avail < kRxMax) {
        uint32_t slot = (e + uint32_t(avail)) % S;
        uint32_t f = ld_acquire_sys(p.in[r].flags + size_t(slot) * p.n_tiles + tile);
        if (f != e + uint32_t(avail) + 1u) break;
        avail++;
      }
      cc[r] = uint8_t((avail << 6) | int(e % S));
      if (avail) work = true;
    }
  }
  if (p.do_tx) {
    for (int r = 0; r < p.n_out; r++) {
      uint32_t t = p.out[r].tx_seq[tile];
      uint32_t c = ld_acquire_sys(p.out[r].credit + tile);
      uint32_t used = t - c;
      uint32_t room = used < S ? S - used : 0u;  // free slots, reported up to 3
      cc[8 + r] = uint8_t((min(room, 3u) << 6) | (t % S));
    }
  }
  *reinterpret_cast<uint4*>(p.ctrl + size_t(tile) * 16) = cur;
  if (work) {
    int idx = atomicAdd(p.work_count + par, 1);
    p.worklist[idx] = tile;
  }
}

// ----------------------------------------------------------------------------------------------
// round_main
// ----------------------------------------------------------------------------------------------
namespace {

// shared -> global bulk store / reduce (this CTA's memory as source), tracked by bulk async-groups
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// barrier over one 128-thread group (hardware barrier 1 + group)
__device__ __forceinline__ void group_bar(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kGroupThreads) : "memory");
}
constexpr uint32_t kFlagChanged = 1, kFlagFailed = 2, kFlagNonsilent0 = 4;  // nonsilent: one bit per pass, 4 << f
constexpr int kMaxFrames = 3;       // 1-bit frames per link, tile and round

// frame words and scale bytes were written by a neighbour GPU: read them from L2, never from this SM's L1
__device__ __forceinline__ uint32_t ld_u32_ca(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_u8_ca(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// f = +/- 2^(code-127) for element `bit` of word w, as raw bits: the sign bit is the frame's bit
__device__ __forceinline__ float signed_scale(uint32_t scale_bits, uint32_t w, int bit) {
  return __uint_as_float(scale_bits | ((w << (31 - bit)) & 0x80000000u));
}

// ---- per-thread arithmetic on 32 consecutive elements held as eight float4 pieces; piece q holds elements
// 4*(q^sw) .. +3.  VMASK: bit i set = element i of the 32 exists (all ones except in a tensor's last chunk).

// a += frame and b += frame with one decode (values and the mirror of the link the frame came from)
template <bool FULL>
__device__ __forceinline__ void apply_frame2(float4 (&a)[8], float4 (&b)[8], uint32_t w, uint32_t sb, int sw, uint32_t vmask) {
#pragma unroll
  for (int q = 0; q < 8; q++) {
    const int sh = 4 * (q ^ sw);
    const uint32_t wq = w >> sh;
    const float f0 = signed_scale(sb, wq, 0), f1 = signed_scale(sb, wq, 1), f2 = signed_scale(sb, wq, 2), f3 = signed_scale(sb, wq, 3);
    if (FULL) {
      a[q].x = __fadd_rn(a[q].x, f0); b[q].x = __fadd_rn(b[q].x, f0);
      a[q].y = __fadd_rn(a[q].y, f1); b[q].y = __fadd_rn(b[q].y, f1);
      a[q].z = __fadd_rn(a[q].z, f2); b[q].z = __fadd_rn(b[q].z, f2);
      a[q].w = __fadd_rn(a[q].w, f3); b[q].w = __fadd_rn(b[q].w, f3);
    } else {
      const uint32_t vq = vmask >> sh;
      if (vq & 1u) { a[q].x = __fadd_rn(a[q].x, f0); b[q].x = __fadd_rn(b[q].x, f0); }
      if (vq & 2u) { a[q].y = __fadd_rn(a[q].y, f1); b[q].y = __fadd_rn(b[q].y, f1); }
      if (vq & 4u) { a[q].z = __fadd_rn(a[q].z, f2); b[q].z = __fadd_rn(b[q].z, f2); }
      if (vq & 8u) { a[q].w = __fadd_rn(a[q].w, f3); b[q].w = __fadd_rn(b[q].w, f3); }
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

// the sign word of v - k (bit i set = element i is not positive) and, if code != 0, the step of the mirror
template <bool FULL>
__device__ __forceinline__ uint32_t sign_word_and_step(const float4 (&v)[8], float4 (&k)[8], uint32_t code, int sw, uint32_t vmask) {
  const float sp = __uint_as_float(code << 23), sn = __uint_as_float((code << 23) | 0x80000000u);
  uint32_t word = 0;
#pragma unroll
  for (int q = 0; q < 8; q++) {
    const int sh = 4 * (q ^ sw);
    const bool n0 = !(__fsub_rn(v[q].x, k[q].x) > 0.f), n1 = !(__fsub_rn(v[q].y, k[q].y) > 0.f);
    const bool n2 = !(__fsub_rn(v[q].z, k[q].z) > 0.f), n3 = !(__fsub_rn(v[q].w, k[q].w) > 0.f);
    uint32_t nib = (n0 ? 1u : 0u) | (n1 ? 2u : 0u) | (n2 ? 4u : 0u) | (n3 ? 8u : 0u);
    if (FULL) {
      if (code) {
        k[q].x = __fadd_rn(k[q].x, n0 ? sn : sp);
        k[q].y = __fadd_rn(k[q].y, n1 ? sn : sp);
        k[q].z = __fadd_rn(k[q].z, n2 ? sn : sp);
        k[q].w = __fadd_rn(k[q].w, n3 ? sn : sp);
      }
    } else {
      const uint32_t vq = (vmask >> sh) & 0xfu;
      nib &= vq;
      if (code) {
        if (vq & 1u) k[q].x = __fadd_rn(k[q].x, n0 ? sn : sp);
        if (vq & 2u) k[q].y = __fadd_rn(k[q].y, n1 ? sn : sp);
        if (vq & 4u) k[q].z = __fadd_rn(k[q].z, n2 ? sn : sp);
        if (vq & 8u) k[q].w = __fadd_rn(k[q].w, n3 ? sn : sp);
      }
    }
    word |= nib << sh;
  }
  return word;
}

struct GroupSmem {
  int off_slots;    // [kGroups][kSlots][kTileBytes]
  int off_vstage;   // [kGroups][kTileBytes]   values of the tile on their way back to global memory
  int off_out;      // [kGroups][2][3 frames][payload_bytes]
  int off_bar;      // uint64_t[kGroups][kSlots]
  int off_red;      // float[kGroups][2][4]   cross-warp partials for blocks of 2048/4096
  int off_flags;    // uint32_t[kGroups][3]  per-step OR flags (changed / nonsilent / wait failed)
  int total;
};
__host__ __device__ inline GroupSmem group_layout(int payload_bytes, int kGroups) {
  GroupSmem m;
  int off = 0;
  m.off_slots = off;
  const int kSlots = slots_for(kGroups);
  off += kGroups * kSlots * kTileBytes;
  m.off_vstage = off;
  off += kGroups * kTileBytes;
  m.off_out = off;
  off += kGroups * 2 * 3 * ((payload_bytes + 127) & ~127);
  m.off_bar = off;
  off += 8 * kGroups * kSlots;
  m.off_red = off;
  off += 4 * kGroups * 2 * 4;
  m.off_flags = off;
  off += 4 * kGroups * 4;
  m.total = (off + 127) & ~127;
  return m;
}

}  // namespace

int round_main_smem_bytes(int, int, int payload_bytes, int* stages_out) {
  if (stages_out) *stages_out = slots_for(3);
  return group_layout(payload_bytes, 3).total;
}

template <int kGroups>
__global__ void __launch_bounds__(kGroups * kGroupThreads, 1) round_main_kernel(const __grid_constant__ RoundParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kSlots = slots_for(kGroups);
  const GroupSmem lay = group_layout(p.payload_bytes, kGroups);
  const int tid = threadIdx.x;
  const int g = tid >> 7;           // group
  const int t = tid & 127;          // thread in group = 32-element chunk of the tile
  const int lane = tid & 31;
  const int wig = (tid >> 5) & 3;   // warp in group
  const int sw = t & 7;             // XOR swizzle of this thread's eight 16-byte pieces
  uint8_t* slots = smem + lay.off_slots + size_t(g) * kSlots * kTileBytes;
  float4* vstage4 = reinterpret_cast<float4*>(smem + lay.off_vstage + size_t(g) * kTileBytes) + t * 8;
  const int pb_pad = (p.payload_bytes + 127) & ~127;
  uint8_t* outbuf = smem + lay.off_out + size_t(g) * 2 * kMaxFrames * pb_pad;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bar) + g * kSlots;
  float* s_red = reinterpret_cast<float*>(smem + lay.off_red) + g * 8;
  uint32_t* s_flags = reinterpret_cast<uint32_t*>(smem + lay.off_flags) + g * 4;

  const int par = p.round & 1;
  const int count = p.work_count[par];
  const int L = p.n_links;
  const int arrays = 1 + L;
  const int lb = p.log2_block;
  const int pb = p.payload_bytes;
  const int64_t n = p.n;
  const int stride = int(gridDim.x) * kGroups;
  const int first = int(blockIdx.x) * kGroups + g;
  const int my_count = count > first ? (count - first + stride - 1) / stride : 0;
  const int total_steps = my_count * arrays;
  const int tpb = lb - 5;           // log2(threads per block)

  if (t == 0) {
    s_flags[0] = s_flags[1] = s_flags[2] = 0;
    for (int s = 0; s < kSlots; s++) mbar_init(full + s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncthreads();

  // ---- copy issue (thread 0 of the group).  Step c = (tile index c / arrays, array c % arrays).
  // The tile ids of this and the next listed tile are kept in registers by every thread.
  int tile_cur = my_count > 0 ? p.worklist[first] : 0;
  int tile_next = my_count > 1 ? p.worklist[first + stride] : 0;
  uint4 cw_cur = my_count > 0 ? *reinterpret_cast<const uint4*>(p.ctrl + size_t(tile_cur) * 16) : make_uint4(0u, 0u, 0u, 0u);
  // Mirrors are visited in link order on even rounds and in reverse order on odd rounds: a frame is applied to the
  // values in its own link's step, so links visited earlier in the same tile forward it one round later, and
  // alternating the order shares that delay out.
  const bool reverse = (p.round & 1) != 0;
  auto link_of = [&](int a) -> int { return reverse ? L - a : a - 1; };
  auto src_of = [&](int tile, int a) -> const float* {
    return (a == 0 ? p.values : p.mirror[link_of(a)]) + size_t(tile) * kTile;
  };
  auto issue_load = [&](int c, int tile) {
    const int s = c % kSlots;
    mbar_expect_tx(full + s, kTileBytes);
    bulk_g2s(slots + size_t(s) * kTileBytes, src_of(tile, c % arrays), kTileBytes, full + s);
  };
  if (t == 0) {
    for (int c = 0; c < kSlots - 1 && c < total_steps; c++) issue_load(c, c / arrays == 0 ? tile_cur : tile_next);
  }

  float res_max0 = 0.f, res_max1 = 0.f, res_max2 = 0.f;  // largest outstanding |residual| per link seen by this thread
  uint32_t n_rx = 0, n_tx = 0, n_blocked = 0, n_pending = 0;
  bool aborted = false;

  for (int i = 0; i < my_count && !aborted; i++) {
    const int tile = tile_cur;
    const int tile_nn = (i + 2 < my_count) ? p.worklist[first + (i + 2) * stride] : 0;  // prefetched two tiles ahead
    const uint4 cw = cw_cur;
    if (i + 1 < my_count) cw_cur = *reinterpret_cast<const uint4*>(p.ctrl + size_t(tile_next) * 16);  // used one tile later
    const uint32_t in_lo = cw.x, in_hi = cw.y, out_lo = cw.z, out_hi = cw.w;
    auto in_byte = [&](int r) -> uint32_t { return ((r < 4 ? in_lo : in_hi) >> ((r & 3) * 8)) & 0xffu; };
    auto out_byte = [&](int r) -> uint32_t { return ((r < 4 ? out_lo : out_hi) >> ((r & 3) * 8)) & 0xffu; };
    const int64_t ebase = int64_t(tile) * kTile + int64_t(t) * 32;
    const bool full_chunk = ebase + 32 <= n;
    const int64_t left = n - ebase;  // elements of this thread's chunk that exist
    const uint32_t vmask = left >= 32 ? 0xffffffffu : (left <= 0 ? 0u : ((1u << int(left)) - 1u));
    const bool rx_any = (in_lo & 0xc0c0c0c0u) != 0 || (in_hi & 0xc0c0c0c0u) != 0;
    bool pend_tile = false;
    uint32_t sent_lo = 0, sent_hi = 0;

    float4 v[8];  // piece q holds elements 4*(q^sw) .. +3 of this thread's 32
    for (int a = 0; a < arrays && !aborted; a++) {
      const int c = i * arrays + a;
      const int s = c % kSlots;
      float4* slot4 = reinterpret_cast<float4*>(slots + size_t(s) * kTileBytes) + t * 8;
      const int l = a == 0 ? -1 : link_of(a);

      // Frames that concern this step: none for the values, the link's own in-rings for a mirror; they are
      // decoded once and added to the mirror and to the values, which stay in registers for the whole tile.
      // (A few hundred bytes per tile, from L1/L2.)  They are fetched three at a time so that their load
      // latencies overlap, the first batch before the wait on the slot.
      int it_r = -1, it_f = 0, it_avail = 0;
      uint32_t it_ib = 0;
      auto next_frame = [&]() -> const uint8_t* {
        if (!rx_any || a == 0) return nullptr;
        while (true) {
          if (it_r >= 0 && it_f < it_avail) {
            const int slot_no = (int(it_ib & 63u) + it_f) & (p.ring_slots - 1);  // ring_slots is a power of two
            it_f++;
            return p.in[it_r].payload + (size_t(slot_no) * p.n_tiles + tile) * pb;
          }
          it_r++;
          if (it_r >= p.n_in) return nullptr;
          it_ib = in_byte(it_r);
          it_avail = p.in[it_r].link != l ? 0 : int(it_ib >> 6);
          it_f = 0;
        }
      };
      const uint8_t *fp0 = next_frame(), *fp1 = fp0 ? next_frame() : nullptr, *fp2 = fp1 ? next_frame() : nullptr;
      uint32_t fw0 = 0, fc0 = 0, fw1 = 0, fc1 = 0, fw2 = 0, fc2 = 0;
      auto load_batch = [&]() {
        if (fp0) { fw0 = ld_u32_ca(fp0 + 4 * t); fc0 = ld_u8_ca(fp0 + 4 * kWordsPerTile + (t >> tpb)); }
        if (fp1) { fw1 = ld_u32_ca(fp1 + 4 * t); fc1 = ld_u8_ca(fp1 + 4 * kWordsPerTile + (t >> tpb)); }
        if (fp2) { fw2 = ld_u32_ca(fp2 + 4 * t); fc2 = ld_u8_ca(fp2 + 4 * kWordsPerTile + (t >> tpb)); }
      };
      load_batch();

      // A wait that runs out does not leave the loop by itself (the group's barrier below needs all 128
      // threads): the thread finishes the step on whatever the slot holds and reports the failure through
      // the step's flags, so that the whole group stops together before anything is stored.
      const bool wait_failed = !mbar_wait_bounded(full + s, uint32_t(c / kSlots) & 1u);
      if (t == 0) s_flags[(c + 1) % 3] = 0;  // flags of the next step; last read two barriers ago
      float4 k[8];
      if (a == 0) {
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = slot4[q ^ sw];
      } else {
#pragma unroll
        for (int q = 0; q < 8; q++) k[q] = slot4[q ^ sw];
      }

      bool changed = false;
      auto apply_one = [&](uint32_t w, uint32_t code) {
        if (t == 0) n_rx++;
        if (!code) return;
        changed = true;
        const uint32_t sb = code << 23;  // bits of 2^(code-127)
        if (full_chunk) apply_frame2<true>(v, k, w, sb, sw, vmask); else apply_frame2<false>(v, k, w, sb, sw, vmask);
      };
      while (fp0) {
        const uint32_t w0 = fw0, c0 = fc0, w1 = fw1, c1 = fc1, w2 = fw2, c2 = fc2;
        const bool h1 = fp1 != nullptr, h2 = fp2 != nullptr;
        fp0 = h2 ? next_frame() : nullptr;   // the next batch goes out before this one is applied
        fp1 = fp0 ? next_frame() : nullptr;
        fp2 = fp1 ? next_frame() : nullptr;
        load_batch();
        apply_one(w0, c0);
        if (h1) apply_one(w1, c1);
        if (h2) apply_one(w2, c2);
      }

      int n_frames = 0;             // frames this step may push: room in every out-ring of the link, at most frames_per_round
      uint32_t nonsilent_mask = 0;  // bit f: this thread's block had something to say in pass f
      if (a > 0) {
        // ---------------- quantise values - mirror for link l, up to frames_per_round times in a row:
        // every pass is one more 1-bit frame of the same stream, made while the data is in registers
        int room = 3;             // free ring slots, the minimum over the link's out-rings
        bool any_ring = false;
        for (int r = 0; r < p.n_out; r++) {
          if (p.out[r].link != l) continue;
          any_ring = true;
          room = min(room, int(out_byte(r) >> 6));
        }
        n_frames = any_ring ? min(room, p.frames_per_round) : 0;
        uint32_t vmax = max_abs_bits(v);
        for (int sft = 0; sft < tpb && sft < 5; sft++) vmax = max(vmax, __shfl_xor_sync(0xffffffffu, vmax, 1 << sft));
        const int passes = n_frames > 0 ? n_frames : 1;  // without ring space one pass still tells whether work is left
        for (int f = 0; f < passes; f++) {
          float xm = residual_maxabs(v, k);
          if (f == 0) {
            if (l == 0) res_max0 = fmaxf(res_max0, xm); else if (l == 1) res_max1 = fmaxf(res_max1, xm); else res_max2 = fmaxf(res_max2, xm);
          }
          // blocks larger than 32 elements: maximum over lanes (up to 1024), then over the group's warps
          for (int sft = 0; sft < tpb && sft < 5; sft++) xm = fmaxf(xm, __shfl_xor_sync(0xffffffffu, xm, 1 << sft));
          uint32_t vm = vmax;
          if (tpb > 5) {
            if (lane == 0) {
              s_red[wig] = xm;
              s_red[4 + wig] = __uint_as_float(vmax);
            }
            group_bar(g);
            const float a0 = s_red[0], a1 = s_red[1], a2 = s_red[2], a3 = s_red[3];
            const uint32_t b0 = __float_as_uint(s_red[4]), b1 = __float_as_uint(s_red[5]);
            const uint32_t b2 = __float_as_uint(s_red[6]), b3 = __float_as_uint(s_red[7]);
            if (tpb == 6) {  // 2048: warps {0,1} and {2,3}
              xm = wig < 2 ? fmaxf(a0, a1) : fmaxf(a2, a3);
              vm = wig < 2 ? max(b0, b1) : max(b2, b3);
            } else {         // 4096: the whole tile
              xm = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
              vm = max(max(b0, b1), max(b2, b3));
            }
            group_bar(g);  // s_red is reused by the next pass
          }
          const int code = block_code_dev(xm, vm, p.min_exp, p.rel_bits);
          if (code) nonsilent_mask |= 1u << f;
          if (n_frames > 0) {
            const uint32_t word = full_chunk ? sign_word_and_step<true>(v, k, uint32_t(code), sw, vmask)
                                             : sign_word_and_step<false>(v, k, uint32_t(code), sw, vmask);
            if (code) changed = true;
            uint8_t* ob = outbuf + size_t((c & 1) * kMaxFrames + f) * pb_pad;
            reinterpret_cast<uint32_t*>(ob)[t] = word;
            if ((t & ((1 << tpb) - 1)) == 0) ob[4 * kWordsPerTile + (t >> tpb)] = uint8_t(code);
          }
        }
      }

      // ---------------- a changed mirror goes back through its slot (the values are written at the end of the tile)
      if (changed && a > 0) {
#pragma unroll
        for (int q = 0; q < 8; q++) slot4[q ^ sw] = k[q];
      }
      // the tile's values leave through a staging buffer after the last mirror (if any frame arrived for the tile)
      const bool store_values = rx_any && a == arrays - 1;
      if (store_values) {
#pragma unroll
        for (int q = 0; q < 8; q++) vstage4[q ^ sw] = v[q];
      }
      fence_async_smem();
      {
        const uint32_t mine = (changed ? kFlagChanged : 0u) | (nonsilent_mask * kFlagNonsilent0) | (wait_failed ? kFlagFailed : 0u);
        const uint32_t warp_bits = __reduce_or_sync(0xffffffffu, mine);
        if (lane == 0 && warp_bits) atomicOr(&s_flags[c % 3], warp_bits);
      }
      group_bar(g);
      const uint32_t step_flags = s_flags[c % 3];
      if (step_flags & kFlagFailed) {
        aborted = true;
        break;
      }
      const bool any_changed = (step_flags & kFlagChanged) != 0;
      const uint32_t ns_bits = step_flags / kFlagNonsilent0;  // bit f: pass f produced a frame worth sending
      // work is left if the last pass still had something to say (or nothing could be sent at all)
      pend_tile |= (ns_bits >> (n_frames > 0 ? n_frames - 1 : 0)) != 0;

      if (t == 0) {
        void* gdst = const_cast<float*>(src_of(tile, a));
        if (any_changed && a > 0) bulk_s2g(gdst, slots + size_t(s) * kTileBytes, kTileBytes);
        if (store_values) bulk_s2g(p.values + size_t(tile) * kTile, smem + lay.off_vstage + size_t(g) * kTileBytes, kTileBytes);
        if (a > 0 && n_frames > 0 && ns_bits) {
          int sent_here = 0;
          for (int f = 0; f < n_frames; f++) {
            if (!((ns_bits >> f) & 1u)) continue;  // an all-silent pass is not a frame
            const uint8_t* ob = outbuf + size_t((c & 1) * kMaxFrames + f) * pb_pad;
            for (int r = 0; r < p.n_out; r++) {
              if (p.out[r].link != l) continue;
              const int slot_no = (int(out_byte(r) & 63u) + sent_here) & (p.ring_slots - 1);
              bulk_s2g(p.out[r].payload_remote + (size_t(slot_no) * p.n_tiles + tile) * pb, ob, uint32_t(pb));
              n_tx++;
            }
            sent_here++;
          }
          for (int r = 0; r < p.n_out; r++) {
            if (p.out[r].link != l) continue;
            if (r < 4) sent_lo |= uint32_t(sent_here) << (r * 8); else sent_hi |= uint32_t(sent_here) << ((r - 4) * 8);
          }
        } else if (a > 0 && ns_bits && p.do_tx) {
          n_blocked++;
        }
        bulk_commit();
        // the slot used one step ago is free once its store (if any) has read it: refill it
        bulk_wait_read_1();
        const int cn = c + kSlots - 1;
        if (cn < total_steps) {
          const int ti = cn / arrays;
          issue_load(cn, ti == i ? tile : (ti == i + 1 ? tile_next : tile_nn));
        }
      }
    }
    if (aborted) break;
    if (t == 0) {
      *reinterpret_cast<uint2*>(p.sent + size_t(tile) * 8) = make_uint2(sent_lo, sent_hi);
      p.tile_state[tile] = uint8_t(pend_tile ? 1 : 0);
      n_pending += pend_tile ? 1 : 0;
    }
    tile_cur = tile_next;
    tile_next = tile_nn;
  }

  if (t == 0) bulk_wait_all();  // every store of this thread has landed before the kernel ends
  if (aborted) {
    // Leave no copy in flight: give outstanding loads a bounded chance to land before the CTA's shared
    // memory is released.
    if (t == 0) {
      atomicOr(reinterpret_cast<unsigned long long*>(p.status + kStErrors), (unsigned long long)kErrBarrierTimeout);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStWaitTimeouts), 1ull);
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2ull * 1000 * 1000) {
      }
    }
    return;
  }

  // ---------------- statistics: one atomic per group and counter
  {
    float a0 = res_max0, a1 = res_max1, a2 = res_max2;
    for (int o = 16; o > 0; o >>= 1) {
      a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, o));
      a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, o));
      a2 = fmaxf(a2, __shfl_xor_sync(0xffffffffu, a2, o));
    }
    if (lane == 0) {  // non-negative floats order like their bit patterns
      if (a0 != 0.f) atomicMax(reinterpret_cast<unsigned long long*>(p.status + kStResidualMax0), (unsigned long long)__float_as_uint(a0));
      if (a1 != 0.f) atomicMax(reinterpret_cast<unsigned long long*>(p.status + kStResidualMax1), (unsigned long long)__float_as_uint(a1));
      if (a2 != 0.f) atomicMax(reinterpret_cast<unsigned long long*>(p.status + kStResidualMax2), (unsigned long long)__float_as_uint(a2));
    }
  }
  if (t == 0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStTilesProcessed), (unsigned long long)my_count);
    if (n_tx) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStFramesSent), (unsigned long long)n_tx);
    if (n_rx) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStFramesRecv), (unsigned long long)n_rx);
    if (n_blocked) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStBlockedNoCredit), (unsigned long long)n_blocked);
    if (n_pending) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStPendingTiles), (unsigned long long)n_pending);
    if (blockIdx.x == 0 && g == 0) {
      const unsigned long long r = atomicAdd(reinterpret_cast<unsigned long long*>(p.status + kStRounds), 1ull);
      p.status[kStLastWorkCount] = uint64_t(count);
      uint64_t* rec = p.status + kStWords + (r % kTraceEntries) * kTraceWords;  // trace ring, read by stats()
      rec[0] = globaltimer_ns();
      rec[1] = r;
      rec[2] = uint64_t(count);
      rec[3] = p.status[kStFramesSent];
    }
  }
}

// ----------------------------------------------------------------------------------------------
// launchers
// ----------------------------------------------------------------------------------------------
int launch_round_begin(const RoundParams& p, void* stream) {
  int blocks = (p.n_tiles + 255) / 256;
  round_begin_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}
int launch_round_publish(const RoundParams& p, void* stream) {
  int blocks = (p.n_tiles + 255) / 256;
  round_publish_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return int(cudaGetLastError());
}

template <int G>
static int launch_main_t(const RoundParams& p, int ctas, cudaStream_t stream) {
  const int smem = group_layout(p.payload_bytes, G).total;
  static int configured_for = -1;  // per instantiation
  if (configured_for < smem) {
    cudaError_t e = cudaFuncSetAttribute(round_main_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return int(e);
    configured_for = smem;
  }
  round_main_kernel<G><<<ctas, G * kGroupThreads, smem, stream>>>(p);
  return int(cudaGetLastError());
}

// The rounds `rounds[0..count)` as one executable graph: begin -> main -> publish of each, chained.  The graph is
// built node by node, not by stream capture: while any stream of a device is capturing, a device-wide
// synchronisation from any other thread (a user's cudaDeviceSynchronize) fails, and the engine thread builds its
// graph at times the user cannot know.
int build_round_graph(const RoundParams* rounds, int count, int ctas, void** exec_out) {
  *exec_out = nullptr;
  constexpr int G = 3;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaGraphCreate(&graph, 0);
  if (e != cudaSuccess) return int(e);
  cudaGraphNode_t prev = nullptr;
  for (int i = 0; i < count && e == cudaSuccess; i++) {
    RoundParams p = rounds[i];
    if (p.n_links < 1 || p.n_links > kMaxLinks) {
      e = cudaErrorInvalidValue;
      break;
    }
    const int smem = group_layout(p.payload_bytes, G).total;
    e = cudaFuncSetAttribute(round_main_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) break;
    void* args[1] = {&p};  // copied into the node when it is added
    const unsigned tile_blocks = unsigned((p.n_tiles + 255) / 256);
    struct {
      void* fn;
      unsigned grid, block, smem;
    } k[3] = {{reinterpret_cast<void*>(round_begin_kernel), tile_blocks, 256u, 0u},
              {reinterpret_cast<void*>(round_main_kernel<G>), unsigned(ctas), unsigned(G * kGroupThreads), unsigned(smem)},
              {reinterpret_cast<void*>(round_publish_kernel), tile_blocks, 256u, 0u}};
    for (int j = 0; j < 3 && e == cudaSuccess; j++) {
      cudaKernelNodeParams np = {};
      np.func = k[j].fn;
      np.gridDim = dim3(k[j].grid);
      np.blockDim = dim3(k[j].block);
      np.sharedMemBytes = k[j].smem;
      np.kernelParams = args;
      np.extra = nullptr;
      cudaGraphNode_t node = nullptr;
      e = cudaGraphAddKernelNode(&node, graph, prev ? &prev : nullptr, prev ? 1 : 0, &np);
      prev = node;
    }
  }
  cudaGraphExec_t exec = nullptr;
  if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return int(e);
  }
  *exec_out = exec;
  return 0;
}

int launch_round_main(const RoundParams& p, int ctas, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.n_links < 1 || p.n_links > kMaxLinks) return int(cudaErrorInvalidValue);
  // 3 groups of 128 threads: 168 registers per thread (no spills) and 3 x (3 slots + staging) x 16 KB of shared memory
  return launch_main_t<3>(p, ctas, stream);
}

}  // namespace st
