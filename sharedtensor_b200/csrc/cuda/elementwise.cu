// Bandwidth kernels around the sync round, sm_100a:
//   snapshot      copyToTensor            out = values                  (reference src/sharedtensor.c:442-444)
//   add / sub_add addFromTensor/pushUpdate values += d | values += a-b  (reference 338-343; one target instead of four)
//   table_scales  per-tensor energies and exponent codes over a flat arena (the reference's README lists
//                 "table sync" with per-tensor magnitudes as a TODO)
//   sample_sqerr  convergence probe for benchmarks and tests
//   delay         device-side pacing
//   snapshot_join values -> a new child's replica and -> the new link's mirror in one pass
//   tensor_*      tensor-scale frames (reference wire format) encoded/decoded on the device for TCP edges
// All are grid-stride kernels with 16-byte accesses sized to 148 SMs; none waits on anything.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "round.h"

namespace st {

namespace {

constexpr int kEwThreads = 256;

inline int ew_blocks(int64_t work_items, int per_sm = 8) {
  int64_t b = (work_items + kEwThreads - 1) / kEwThreads;
  int64_t cap = 148 * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

__device__ __forceinline__ float4 ldg_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void red_add_v4(float* p, float4 d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(d.x), "f"(d.y), "f"(d.z), "f"(d.w) : "memory");
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// ---------------------------------------------------------------------------------------------
// snapshot
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kEwThreads) snapshot_f32_vec(const float4* __restrict__ src, float4* __restrict__ dst, int64_t n4) {
  int64_t i = int64_t(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kEwThreads;
  // four independent 16-byte loads in flight per thread
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    __stcs(dst + i, a);
    __stcs(dst + i + stride, b);
    __stcs(dst + i + 2 * stride, c);
    __stcs(dst + i + 3 * stride, d);
  }
  for (; i < n4; i += stride) __stcs(dst + i, src[i]);
}
__global__ void snapshot_f32_scalar(const float* __restrict__ src, float* __restrict__ dst, int64_t begin, int64_t n) {
  int64_t i = begin + int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) dst[i] = src[i];
}
__global__ void __launch_bounds__(kEwThreads) snapshot_bf16_vec(const float4* __restrict__ src, uint2* __restrict__ dst, int64_t n4) {
  int64_t i = int64_t(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kEwThreads;
  for (; i < n4; i += stride) {
    float4 a = src[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    dst[i] = o;
  }
}
__global__ void snapshot_bf16_scalar(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t begin, int64_t n) {
  int64_t i = begin + int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

int launch_snapshot_f32(const float* values, float* out, int64_t n, void* stream_v) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_v);
  int64_t n4 = aligned16(out) && aligned16(values) ? n / 4 : 0;
  if (n4) snapshot_f32_vec<<<ew_blocks(n4 / 4 + 1), kEwThreads, 0, s>>>(reinterpret_cast<const float4*>(values), reinterpret_cast<float4*>(out), n4);
  if (n4 * 4 < n) snapshot_f32_scalar<<<ew_blocks(n - n4 * 4), kEwThreads, 0, s>>>(values, out, n4 * 4, n);
  return int(cudaGetLastError());
}
int launch_snapshot_bf16(const float* values, void* out, int64_t n, void* stream_v) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_v);
  bool al = aligned16(values) && (reinterpret_cast<uintptr_t>(out) & 7) == 0;
  int64_t n4 = al ? n / 4 : 0;
  if (n4) snapshot_bf16_vec<<<ew_blocks(n4), kEwThreads, 0, s>>>(reinterpret_cast<const float4*>(values), reinterpret_cast<uint2*>(out), n4);
  if (n4 * 4 < n) snapshot_bf16_scalar<<<ew_blocks(n - n4 * 4), kEwThreads, 0, s>>>(values, static_cast<__nv_bfloat16*>(out), n4 * 4, n);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// add / sub_add
// ---------------------------------------------------------------------------------------------
template <bool SUB, bool ATOMIC>
__global__ void __launch_bounds__(kEwThreads) add_vec(float4* __restrict__ values, const float4* __restrict__ a, const float4* __restrict__ b,
                                                      int64_t n4) {
  int64_t i = int64_t(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kEwThreads;
  // four independent 16-byte streams per thread and iteration
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 d[4], v[4];
#pragma unroll
    for (int u = 0; u < 4; u++) d[u] = ldg_stream(a + i + u * stride);
    if (SUB) {
#pragma unroll
      for (int u = 0; u < 4; u++) {
        float4 o = ldg_stream(b + i + u * stride);
        d[u].x -= o.x; d[u].y -= o.y; d[u].z -= o.z; d[u].w -= o.w;
      }
    }
    if (ATOMIC) {
#pragma unroll
      for (int u = 0; u < 4; u++) red_add_v4(reinterpret_cast<float*>(values + i + u * stride), d[u]);
    } else {
#pragma unroll
      for (int u = 0; u < 4; u++) v[u] = values[i + u * stride];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        v[u].x += d[u].x; v[u].y += d[u].y; v[u].z += d[u].z; v[u].w += d[u].w;
        values[i + u * stride] = v[u];
      }
    }
  }
  for (; i < n4; i += stride) {
    float4 d0 = ldg_stream(a + i);
    if (SUB) {
      float4 o0 = ldg_stream(b + i);
      d0.x -= o0.x; d0.y -= o0.y; d0.z -= o0.z; d0.w -= o0.w;
    }
    if (ATOMIC) {
      red_add_v4(reinterpret_cast<float*>(values + i), d0);
    } else {
      float4 v0 = values[i];
      v0.x += d0.x; v0.y += d0.y; v0.z += d0.z; v0.w += d0.w;
      values[i] = v0;
    }
  }
}
template <bool SUB, bool ATOMIC>
__global__ void add_scalar(float* __restrict__ values, const float* __restrict__ a, const float* __restrict__ b, int64_t begin, int64_t n) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (i += begin; i < n; i += stride) {
    float d = SUB ? a[i] - b[i] : a[i];
    if (ATOMIC)
      atomicAdd(values + i, d);
    else
      values[i] += d;
  }
}

template <bool SUB>
static int launch_add_t(float* values, const float* a, const float* b, int64_t n, int atomic, cudaStream_t s) {
  bool al = aligned16(values) && aligned16(a) && (!SUB || aligned16(b));
  int64_t n4 = al ? n / 4 : 0;
  if (n4) {
    int blocks = ew_blocks(n4 / 4 + 1);
    if (atomic)
      add_vec<SUB, true><<<blocks, kEwThreads, 0, s>>>(reinterpret_cast<float4*>(values), reinterpret_cast<const float4*>(a),
                                                       reinterpret_cast<const float4*>(b), n4);
    else
      add_vec<SUB, false><<<blocks, kEwThreads, 0, s>>>(reinterpret_cast<float4*>(values), reinterpret_cast<const float4*>(a),
                                                        reinterpret_cast<const float4*>(b), n4);
  }
  if (n4 * 4 < n) {
    int blocks = ew_blocks(n - n4 * 4);
    if (atomic)
      add_scalar<SUB, true><<<blocks, kEwThreads, 0, s>>>(values, a, b, n4 * 4, n);
    else
      add_scalar<SUB, false><<<blocks, kEwThreads, 0, s>>>(values, a, b, n4 * 4, n);
  }
  return int(cudaGetLastError());
}

int launch_add(float* values, const float* delta, int64_t n, int atomic, void* stream) {
  return launch_add_t<false>(values, delta, nullptr, n, atomic, static_cast<cudaStream_t>(stream));
}
int launch_sub_add(float* values, const float* neu, const float* old, int64_t n, int atomic, void* stream) {
  return launch_add_t<true>(values, neu, old, n, atomic, static_cast<cudaStream_t>(stream));
}

// values += alpha * g for a bf16 gradient: the optimiser step of plain SGD fused with addFromTensor, so
// that bf16 training never materialises an fp32 delta.
template <bool ATOMIC>
__global__ void __launch_bounds__(kEwThreads) add_scaled_bf16_vec(float4* __restrict__ values, const uint2* __restrict__ g, float alpha,
                                                                  int64_t n4) {
  int64_t i = int64_t(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kEwThreads;
  for (; i < n4; i += stride) {
    uint2 raw = g[i];
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    if (ATOMIC) {
      red_add_v4(reinterpret_cast<float*>(values + i), make_float4(alpha * a.x, alpha * a.y, alpha * b.x, alpha * b.y));
    } else {
      float4 v = values[i];
      v.x += alpha * a.x;
      v.y += alpha * a.y;
      v.z += alpha * b.x;
      v.w += alpha * b.y;
      values[i] = v;
    }
  }
}
template <bool ATOMIC>
__global__ void add_scaled_bf16_scalar(float* __restrict__ values, const __nv_bfloat16* __restrict__ g, float alpha, int64_t begin,
                                       int64_t n) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (i += begin; i < n; i += stride) {
    if (ATOMIC) atomicAdd(values + i, alpha * __bfloat162float(g[i]));
    else values[i] += alpha * __bfloat162float(g[i]);
  }
}
int launch_add_scaled_bf16(float* values, const void* g_bf16, float alpha, int64_t n, int atomic, void* stream_v) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_v);
  bool al = aligned16(values) && (reinterpret_cast<uintptr_t>(g_bf16) & 7) == 0;
  int64_t n4 = al ? n / 4 : 0;
  if (n4) {
    if (atomic) add_scaled_bf16_vec<true><<<ew_blocks(n4), kEwThreads, 0, s>>>(reinterpret_cast<float4*>(values), static_cast<const uint2*>(g_bf16), alpha, n4);
    else add_scaled_bf16_vec<false><<<ew_blocks(n4), kEwThreads, 0, s>>>(reinterpret_cast<float4*>(values), static_cast<const uint2*>(g_bf16), alpha, n4);
  }
  if (n4 * 4 < n) {
    if (atomic) add_scaled_bf16_scalar<true><<<ew_blocks(n - n4 * 4), kEwThreads, 0, s>>>(values, static_cast<const __nv_bfloat16*>(g_bf16), alpha, n4 * 4, n);
    else add_scaled_bf16_scalar<false><<<ew_blocks(n - n4 * 4), kEwThreads, 0, s>>>(values, static_cast<const __nv_bfloat16*>(g_bf16), alpha, n4 * 4, n);
  }
  return int(cudaGetLastError());
}

__global__ void fill_state_kernel(uint32_t* s, int n, uint32_t v) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) s[i] = v;
}
__global__ void set_word_kernel(uint32_t* w, uint32_t v) { *w = v; }
int launch_set_word(uint32_t* word, uint32_t value, void* stream) {
  set_word_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(word, value);
  return int(cudaGetLastError());
}
int launch_fill_state(uint32_t* tile_state, int n_tiles, uint32_t value, void* stream) {
  fill_state_kernel<<<(n_tiles + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(tile_state, n_tiles, value);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// table_scales: two passes.  Pass 1: every CTA owns a contiguous chunk of one segment and writes one
// partial sum (double) into scratch.  Pass 2: one warp per segment adds that segment's partials in a
// fixed order (deterministic result) and derives the exponent code of the segment's RMS.
// ---------------------------------------------------------------------------------------------
constexpr int64_t kTsChunk = 1 << 16;  // elements per pass-1 CTA

int64_t table_scales_scratch_doubles(int n_seg, int64_t n_total) { return n_total / kTsChunk + 2 * int64_t(n_seg) + 2; }

// chunk c of the arena's chunk list: segment s covers chunks [first[s], first[s+1]).  A CTA walks over every
// gridDim.x-th chunk; a thread keeps four independent 16-byte loads in flight and four independent sums.
__global__ void __launch_bounds__(256) table_partial_kernel(const float* __restrict__ x, const int64_t* __restrict__ off, int n_seg,
                                                            const int64_t* __restrict__ first_chunk, double* __restrict__ partials,
                                                            int64_t max_chunks) {
  __shared__ double red[8];
  __shared__ int s_seg;
  int64_t n_chunks = first_chunk[n_seg];
  if (n_chunks > max_chunks) n_chunks = max_chunks;  // an inconsistent table never reaches past the scratch buffer
  for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    if (threadIdx.x == 0) {
      int lo = 0, hi = n_seg - 1;  // last segment whose first chunk is <= c
      while (lo < hi) {
        int mid = (lo + hi + 1) / 2;
        if (first_chunk[mid] <= c) lo = mid; else hi = mid - 1;
      }
      s_seg = lo;
    }
    __syncthreads();
    const int seg = s_seg;
    const int64_t begin = off[seg] + (c - first_chunk[seg]) * kTsChunk;
    const int64_t end = min(begin + kTsChunk, off[seg + 1]);
    double acc = 0.0;
    // 16-byte loads over the aligned middle of the chunk, scalar loads at its ragged ends
    int64_t a0 = (begin + 3) & ~int64_t(3);
    if (a0 > end) a0 = end;
    const int64_t a1 = a0 + ((end - a0) & ~int64_t(3));
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      for (int64_t i = begin + threadIdx.x; i < a0; i += 256) acc += double(x[i]) * double(x[i]);
      const float4* x4 = reinterpret_cast<const float4*>(x);
      const int64_t q1 = a1 / 4;
      int64_t i = a0 / 4 + threadIdx.x;
      double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
      for (; i + 768 < q1; i += 1024) {
        const float4 v0 = ldg_stream(x4 + i), v1 = ldg_stream(x4 + i + 256), v2 = ldg_stream(x4 + i + 512), v3 = ldg_stream(x4 + i + 768);
        s0 += (double(v0.x) * double(v0.x) + double(v0.y) * double(v0.y)) + (double(v0.z) * double(v0.z) + double(v0.w) * double(v0.w));
        s1 += (double(v1.x) * double(v1.x) + double(v1.y) * double(v1.y)) + (double(v1.z) * double(v1.z) + double(v1.w) * double(v1.w));
        s2 += (double(v2.x) * double(v2.x) + double(v2.y) * double(v2.y)) + (double(v2.z) * double(v2.z) + double(v2.w) * double(v2.w));
        s3 += (double(v3.x) * double(v3.x) + double(v3.y) * double(v3.y)) + (double(v3.z) * double(v3.z) + double(v3.w) * double(v3.w));
      }
      for (; i < q1; i += 256) {
        const float4 v = ldg_stream(x4 + i);
        s0 += (double(v.x) * double(v.x) + double(v.y) * double(v.y)) + (double(v.z) * double(v.z) + double(v.w) * double(v.w));
      }
      acc += (s0 + s1) + (s2 + s3);
      for (int64_t j = a1 + threadIdx.x; j < end; j += 256) acc += double(x[j]) * double(x[j]);
    } else {
      for (int64_t i = begin + threadIdx.x; i < end; i += 256) {
        float v = x[i];
        acc += double(v) * double(v);
      }
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int w = 0; w < 8; w++) t += red[w];
      partials[c] = t;
    }
    __syncthreads();  // red and s_seg are reused by the next chunk
  }
}
__global__ void table_final_kernel(const int64_t* __restrict__ off, int n_seg, const int64_t* __restrict__ first_chunk,
                                   const double* __restrict__ partials, double* __restrict__ out_sumsq, int8_t* __restrict__ out_exp,
                                   int64_t max_chunks) {
  int seg = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  if (seg >= n_seg) return;
  const int lane = threadIdx.x & 31;
  double acc = 0.0;
  const int64_t c0 = first_chunk[seg], c1 = first_chunk[seg + 1];
  const bool consistent = c0 >= 0 && c0 <= c1 && c1 <= max_chunks;  // offsets that ascend and end where the caller said
  if (consistent)
    for (int64_t c = c0 + lane; c < c1; c += 32) acc += partials[c];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    int64_t cnt = off[seg + 1] - off[seg];
    int e = -128;
    if (!consistent) {
      acc = __longlong_as_double(0x7ff8000000000000LL);  // NaN: the table contradicts n_total
    } else if (cnt > 0 && acc > 0.0) {
      double rms = sqrt(acc / double(cnt));
      int ex;
      frexp(rms, &ex);
      e = ex - 1;
      if (e < -126) e = -128;
      if (e > 127) e = 127;
    }
    out_sumsq[seg] = acc;
    out_exp[seg] = int8_t(e);
  }
}
__global__ void table_chunks_kernel(const int64_t* __restrict__ off, int n_seg, int64_t* __restrict__ first_chunk) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int64_t c = 0;
    for (int s = 0; s < n_seg; s++) {
      first_chunk[s] = c;
      const int64_t len = off[s + 1] - off[s];
      c += len > 0 ? (len + kTsChunk - 1) / kTsChunk : 0;
    }
    first_chunk[n_seg] = c;
  }
}

int launch_table_scales(const float* x, const int64_t* seg_offsets_dev, int n_seg, int64_t n_total, double* scratch, double* out_sumsq,
                        int8_t* out_exp, void* stream_v) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_v);
  // scratch layout: [first_chunk: n_seg+1 int64][partials: up to n_total/chunk + n_seg doubles]
  int64_t* first_chunk = reinterpret_cast<int64_t*>(scratch);
  double* partials = scratch + (n_seg + 1);
  const int64_t max_chunks = n_total / kTsChunk + n_seg;  // holds for offsets that ascend from 0 to n_total
  table_chunks_kernel<<<1, 32, 0, s>>>(seg_offsets_dev, n_seg, first_chunk);
  // the exact chunk count lives on the device: a grid of at most eight CTAs per SM walks over the chunks there are
  const int64_t grid = max_chunks < 148 * 8 ? (max_chunks < 1 ? 1 : max_chunks) : 148 * 8;
  table_partial_kernel<<<unsigned(grid), 256, 0, s>>>(x, seg_offsets_dev, n_seg, first_chunk, partials, max_chunks);
  table_final_kernel<<<(n_seg + 7) / 8, 256, 0, s>>>(seg_offsets_dev, n_seg, first_chunk, partials, out_sumsq, out_exp, max_chunks);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// sample_sqerr / delay / snapshot_join
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sample_sqerr_kernel(const float* __restrict__ a, int64_t stride_a, const float* __restrict__ b,
                                                           int64_t count, double* __restrict__ out) {
  double acc = 0.0;
  unsigned long long nan = 0;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < count; i += int64_t(gridDim.x) * 256) {
    float d = a[i * stride_a] - b[i];
    if (d != d) nan++;
    acc += double(d) * double(d);
  }
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
    nan += __shfl_xor_sync(0xffffffffu, nan, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out, acc);
    if (nan) atomicAdd(reinterpret_cast<unsigned long long*>(out + 1), nan);
  }
}
int launch_sample_sqerr(const float* a, int64_t stride, const float* b, int64_t count, double* out, void* stream) {
  sample_sqerr_kernel<<<ew_blocks(count, 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, stride, b, count, out);
  return int(cudaGetLastError());
}

// Convergence probe with a device time stamp: the sampled squared error of `a` against `b`, and when it is at or
// below `threshold` for the first time, the GPU's clock into *stamp (left alone once it is non-zero).  scratch:
// one double (the running sum, left at zero for the next launch) and one counter word behind it.
__global__ void __launch_bounds__(256) probe_converged_kernel(const float* __restrict__ a, int64_t stride_a, const float* __restrict__ b,
                                                              int64_t count, double threshold, double* __restrict__ scratch,
                                                              unsigned long long* __restrict__ stamp, double* __restrict__ last_err) {
  double acc = 0.0;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < count; i += int64_t(gridDim.x) * 256) {
    float d = a[i * stride_a] - b[i];
    acc += double(d) * double(d);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ double part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < 8; w++) t += part[w];
    atomicAdd(scratch, t);
    __threadfence();
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch + 1);
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {  // the last block: every partial sum is in
      const double total = atomicAdd(scratch, 0.0);
      *last_err = total;
      if (total <= threshold && *stamp == 0ull) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        *stamp = now;
      }
      *scratch = 0.0;
      *counter = 0u;
      __threadfence();
    }
  }
}
int launch_probe_converged(const float* a, int64_t stride, const float* b, int64_t count, double threshold, double* scratch,
                           uint64_t* stamp, double* last_err, void* stream) {
  probe_converged_kernel<<<ew_blocks(count, 2), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, stride, b, count, threshold, scratch, reinterpret_cast<unsigned long long*>(stamp), last_err);
  return int(cudaGetLastError());
}
// The GPU's clock into *out: launched behind an update it marks the moment the update had landed; launched alone and
// timed from the host it relates the GPU's clock to the host's.
__global__ void stamp_kernel(unsigned long long* out) {
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  *out = now;
}
int launch_stamp(uint64_t* out, void* stream) {
  stamp_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<unsigned long long*>(out));
  return int(cudaGetLastError());
}

__global__ void delay_kernel(uint64_t ns) {
  uint64_t t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  // bounded by construction: the loop ends when the clock passes t0 + ns, and by an iteration cap
  for (uint64_t it = 0; it < (1ull << 32); it++) {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 >= ns) break;
    __nanosleep(200);
  }
}
int launch_delay(uint64_t ns, void* stream) {
  if (ns > 1000ull * 1000 * 1000) ns = 1000ull * 1000 * 1000;  // never longer than a second
  delay_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(ns);
  return int(cudaGetLastError());
}

__global__ void __launch_bounds__(kEwThreads) snapshot_join_kernel(const float4* __restrict__ values, float4* __restrict__ dst,
                                                                   float4* __restrict__ mirror, int64_t n4) {
  int64_t i = int64_t(blockIdx.x) * kEwThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kEwThreads;
  for (; i < n4; i += stride) {
    float4 v = values[i];
    dst[i] = v;
    mirror[i] = v;
  }
}
int launch_snapshot_join(const float* values, float* dst_values, float* mirror, int64_t n_padded, void* stream) {
  int64_t n4 = n_padded / 4;
  snapshot_join_kernel<<<ew_blocks(n4), kEwThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(values), reinterpret_cast<float4*>(dst_values), reinterpret_cast<float4*>(mirror), n4);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// tensor-scale frames on the device (one scale for the whole tensor, 1 bit per element)
// ---------------------------------------------------------------------------------------------
// out2[0] = bits of max |v - k|, out2[1] = bits of max |v| (non-negative floats order like their bit patterns)
__global__ void __launch_bounds__(256) tensor_maxabs_kernel(const float* __restrict__ v, const float* __restrict__ k, int64_t n,
                                                            uint32_t* __restrict__ out2) {
  float mx = 0.f, mv = 0.f;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n; i += int64_t(gridDim.x) * 256) {
    float a = v[i];
    mx = fmaxf(mx, fabsf(a - k[i]));
    mv = fmaxf(mv, fabsf(a));
  }
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(out2, __float_as_uint(mx));
    atomicMax(out2 + 1, __float_as_uint(mv));
  }
}
int launch_tensor_maxabs(const float* v, const float* k, int64_t n, uint32_t* out2, void* stream) {
  tensor_maxabs_kernel<<<ew_blocks(n, 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(v, k, n, out2);
  return int(cudaGetLastError());
}
// words[i/32] bit i%32 = !(v-k > 0); k steps by -/+ scale.  n is padded by the caller to a multiple of 32
// with v = k = 0 beyond the valid range; `n_valid` stops the mirror update there.
__global__ void __launch_bounds__(256) tensor_encode_kernel(const float* __restrict__ v, float* __restrict__ k, int64_t n_valid, float scale,
                                                            uint32_t* __restrict__ words, int64_t n_words) {
  const int lane = threadIdx.x & 31;
  for (int64_t w = (int64_t(blockIdx.x) * 256 + threadIdx.x) >> 5; w < n_words; w += (int64_t(gridDim.x) * 256) >> 5) {
    int64_t i = w * 32 + lane;
    bool valid = i < n_valid;
    float kk = valid ? k[i] : 0.f;
    float x = valid ? v[i] - kk : 0.f;
    bool neg = valid && !(x > 0.f);
    uint32_t word = __ballot_sync(0xffffffffu, neg);
    if (valid && scale != 0.f) k[i] = kk + (neg ? -scale : scale);
    if (lane == 0) words[w] = word;
  }
}
int launch_tensor_encode(const float* v, float* k, int64_t n, float scale, uint32_t* words, void* stream) {
  int64_t n_words = (n + 31) / 32;
  tensor_encode_kernel<<<ew_blocks(n_words * 32, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(v, k, n, scale, words, n_words);
  return int(cudaGetLastError());
}
template <bool ATOMIC>
__global__ void __launch_bounds__(256) tensor_decode_kernel(const uint32_t* __restrict__ words, float scale, int64_t n, float* __restrict__ v,
                                                            float* __restrict__ k) {
  int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * 256;
  for (; i < n; i += stride) {
    float f = ((words[i >> 5] >> (i & 31)) & 1u) ? -scale : scale;
    if (ATOMIC) atomicAdd(v + i, f);
    else v[i] += f;
    if (k) k[i] += f;
  }
}
int launch_tensor_decode(const uint32_t* words, float scale, int64_t n, float* v, float* k, int atomic_v, void* stream) {
  if (scale == 0.f) return 0;
  if (atomic_v) tensor_decode_kernel<true><<<ew_blocks(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(words, scale, n, v, k);
  else tensor_decode_kernel<false><<<ew_blocks(n, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(words, scale, n, v, k);
  return int(cudaGetLastError());
}

}  // namespace st
