/* Per-tensor energies of a table of tensors, for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference (which has neither GPU code nor table sync).
 *
 * Who needs it: code that runs where a device allocation is off the table.  Two examples are a job whose
 * memory pool has taken all of the GPU, so that a cudaMalloc for a few kilobytes of scratch fails, and a
 * monitoring hook inside a latency-critical loop, where cudaMalloc/cudaFree would quietly synchronise the
 * whole device.  The ordinary path (launch_table_scales in round.h) leaves the scratch buffer to its
 * caller; this one brings its own: a fixed 512 KiB array that lives in the library's device image.  Every
 * GPU that loads the library carries that array until the process ends, whether or not this function is
 * ever called.
 *
 * The function calls no cudaMalloc, cudaFree or other allocating routine.  The caller still owns and
 * passes every input and output.
 *
 * Limits (checked, see the error codes): at most ST_NOALLOC_MAX_SEGMENTS tensors and
 * ST_NOALLOC_MAX_ELEMENTS elements in total.  The offsets live on the device, so the host cannot check them:
 * n_total has to be the last offset and the offsets have to ascend.  A table that contradicts n_total never
 * makes the kernels reach past the scratch array; the tensors concerned come back with NaN as their energy.
 *
 * First call on a device: the address of the array on the CURRENT device is looked up once
 * (cudaGetSymbolAddress) and remembered.  Make that first call with the right device current and before
 * starting any stream capture on it.
 *
 * Sharing: all calls on a device use the same array, and it keeps whatever the previous call left in it.
 * Nothing in it has to start at zero (each call writes every word before reading it), but two calls that
 * overlap on the GPU, on different streams for instance, overwrite each other's partial sums and both
 * produce garbage.  Put them on one stream or order them with events.
 */
#ifndef SHAREDTENSOR_B200_NOALLOC_H
#define SHAREDTENSOR_B200_NOALLOC_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ST_NOALLOC_MAX_SEGMENTS 4096
#define ST_NOALLOC_MAX_ELEMENTS 2147483648LL /* 2^31 */
#define ST_NOALLOC_SCRATCH_BYTES (512 * 1024)

enum {
  ST_NOALLOC_OK = 0,
  ST_NOALLOC_TOO_MANY_SEGMENTS = -1, /* n_seg outside 1..ST_NOALLOC_MAX_SEGMENTS */
  ST_NOALLOC_TOO_MANY_ELEMENTS = -2, /* n_total outside 0..ST_NOALLOC_MAX_ELEMENTS */
  ST_NOALLOC_BAD_ARGUMENT = -3,      /* a null pointer */
  ST_NOALLOC_CUDA_ERROR = -4         /* device lookup, symbol lookup or launch failed; see st_noalloc_last_cuda_error */
};

/* x: device, n_total floats (the arena).  seg_offsets: device, n_seg+1 int64, ascending, first 0, last n_total.
 * out_sumsq: device, n_seg doubles (sum of squares per tensor).  out_exp: device, n_seg int8
 * (floor(log2(rms)) per tensor, -128 for an empty or all-zero tensor).  stream: a cudaStream_t.
 * Asynchronous: results are ready when the stream reaches the end of the three kernels it enqueues. */
int st_table_scales_noalloc(const float* x, const int64_t* seg_offsets, int n_seg, int64_t n_total, double* out_sumsq,
                            int8_t* out_exp, void* stream);

/* The cudaError_t behind the last ST_NOALLOC_CUDA_ERROR of this thread (0 if none). */
int st_noalloc_last_cuda_error(void);
const char* st_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
