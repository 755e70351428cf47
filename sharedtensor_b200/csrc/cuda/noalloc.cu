// Allocation-free variant of the table-scales kernels: same kernels, scratch taken from a static device
// array instead of a caller-provided buffer.  See noalloc.h for who this is for and for the rules.
#include "noalloc.h"

#include <cuda_runtime.h>

#include <mutex>

#include "round.h"

namespace {

// The scratch: first_chunk table (n_seg+1 int64) followed by one partial sum per 65536-element chunk.
// 512 KiB = 65536 doubles covers 4096 tensors and 2^31 elements (4097 + 32768 + 4096 words) with room to spare.
static __device__ __align__(256) double g_noalloc_scratch[ST_NOALLOC_SCRATCH_BYTES / sizeof(double)];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
double* g_scratch_on_device[kMaxDevices];  // device address of g_noalloc_scratch per device ordinal, looked up once
thread_local int t_last_cuda_error = 0;

}  // namespace

#define ST_EXPORT extern "C" __attribute__((visibility("default")))

ST_EXPORT int st_table_scales_noalloc(const float* x, const int64_t* seg_offsets, int n_seg, int64_t n_total, double* out_sumsq,
                                      int8_t* out_exp, void* stream) {
  if (n_seg < 1 || n_seg > ST_NOALLOC_MAX_SEGMENTS) return ST_NOALLOC_TOO_MANY_SEGMENTS;
  if (n_total < 0 || n_total > ST_NOALLOC_MAX_ELEMENTS) return ST_NOALLOC_TOO_MANY_ELEMENTS;
  if (!seg_offsets || !out_sumsq || !out_exp || (!x && n_total > 0)) return ST_NOALLOC_BAD_ARGUMENT;
  if (st::table_scales_scratch_doubles(n_seg, n_total) > int64_t(ST_NOALLOC_SCRATCH_BYTES / sizeof(double)))
    return ST_NOALLOC_TOO_MANY_ELEMENTS;  // cannot happen within the two limits above; kept as a guard

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    t_last_cuda_error = int(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return ST_NOALLOC_CUDA_ERROR;
  }
  double* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(g_mu);
    scratch = g_scratch_on_device[dev];
    if (!scratch) {
      // In host code `g_noalloc_scratch` is only a handle for the symbol, not an address a kernel could use.
      // The device address on the current device comes from the runtime, once per device.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p) {
        t_last_cuda_error = int(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
        return ST_NOALLOC_CUDA_ERROR;
      }
      scratch = static_cast<double*>(p);
      g_scratch_on_device[dev] = scratch;
    }
  }
  // The kernels write the chunk table and every partial sum they later read, so nothing needs clearing.
  int rc = st::launch_table_scales(x, seg_offsets, n_seg, n_total, scratch, out_sumsq, out_exp, stream);
  if (rc != 0) {
    t_last_cuda_error = rc;
    return ST_NOALLOC_CUDA_ERROR;
  }
  return ST_NOALLOC_OK;
}

ST_EXPORT int st_noalloc_last_cuda_error(void) { return t_last_cuda_error; }

ST_EXPORT const char* st_noalloc_strerror(int code) {
  switch (code) {
    case ST_NOALLOC_OK: return "ok";
    case ST_NOALLOC_TOO_MANY_SEGMENTS: return "number of tensors outside 1..4096: the built-in scratch array cannot hold their table";
    case ST_NOALLOC_TOO_MANY_ELEMENTS: return "total element count outside 0..2^31: the built-in scratch array cannot hold the partial sums";
    case ST_NOALLOC_BAD_ARGUMENT: return "null pointer argument";
    case ST_NOALLOC_CUDA_ERROR: return "CUDA call failed (see st_noalloc_last_cuda_error)";
    default: return "unknown code";
  }
}
