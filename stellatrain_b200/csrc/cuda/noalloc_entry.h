// Exact top-k selection of one flat fp32 array for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine.  It exists for callers that cannot
// call cudaMalloc (or any allocator that may end up there): code running inside a memory pool whose
// budget is fixed up front, plugins loaded into a host process that owns all device memory, and
// code on a latency path where an allocation could block behind other work on the device.  They
// hand in the input and the output buffers; every byte of working memory the selection needs
// (histogram, work tables, candidate list, a private copy of the values) lives in one array that
// is part of this library's device image.
//
// Cost of that design, to be known by the user:
//   * the array is ST_NOALLOC_SCRATCH_BYTES large and every GPU on which the library is loaded
//     keeps it resident until the process exits, whether or not the function is ever called;
//   * inputs longer than ST_NOALLOC_MAX_ELEMS are refused with ST_NOALLOC_ERR_TOO_LARGE;
//   * all calls on one GPU share the array.  A call clears what it needs cleared, so calls may
//     follow one another freely on ONE stream, but two calls that overlap on the GPU (different
//     streams, different host threads) race on the array and return garbage;
//   * the first call on each GPU looks up the array's device address.  Make that first call
//     outside of any stream capture.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define ST_NOALLOC_MAX_ELEMS (1u << 20)
#define ST_NOALLOC_SCRATCH_BYTES (13u << 20)

#define ST_NOALLOC_OK 0
#define ST_NOALLOC_ERR_TOO_LARGE 1   // n > ST_NOALLOC_MAX_ELEMS
#define ST_NOALLOC_ERR_BAD_ARG 2     // null pointer, k == 0, k > n, or a misaligned buffer
#define ST_NOALLOC_ERR_CUDA 3        // a CUDA runtime call failed; see st_noalloc_last_error()

#ifdef __cplusplus
extern "C" {
#endif

// Writes the k entries of `values[0..n)` with the largest magnitude to `out_pairs` as k pairs
// {uint32 index, float value bits}; equal magnitudes are resolved towards the lower index; the order
// of the pairs is unspecified; a NaN in the input is treated as 0.  `values` is only read.  `values` must be
// 4-byte and `out_pairs` 8-byte aligned device pointers.  Work is enqueued on `stream`; the
// function does not synchronize.  Returns one of the ST_NOALLOC_* codes.
__attribute__((visibility("default")))
int st_topk_select_noalloc(const float* values, uint32_t n, uint32_t k, void* out_pairs, cudaStream_t stream);

// The selection runs asynchronously, so st_topk_select_noalloc returns before its kernels have run and cannot say
// how they fared.  This call waits for `stream` and copies the device-side status word of the latest selection on
// the current GPU into *status_out (host memory): 0 = the k pairs were written, anything else = the kernels gave
// up and out_pairs is not valid (values of st::Status in sparse_types.h; with well-formed arguments this does not
// happen).  It allocates nothing.  Returns one of the ST_NOALLOC_* codes.
__attribute__((visibility("default")))
int st_noalloc_status(uint32_t* status_out, cudaStream_t stream);

// Human-readable reason of the calling thread's last non-zero return value.
__attribute__((visibility("default")))
const char* st_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
