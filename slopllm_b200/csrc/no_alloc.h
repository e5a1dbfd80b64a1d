// Allocation-free entry point (this has no counterpart in the reference).
//
// Some callers of this library cannot obtain device memory at call time: a plain C or FFI host
// that links the kernels without PyTorch's caching allocator, a serving loop that has handed all
// free HBM to the KV cache, or code that runs while a stream is being captured (cudaMalloc is
// not permitted there).  For them the vocabulary arg-max is offered in a form whose scratch
// space lives inside the library image instead of being passed in.
//
//   int sl_argmax_noalloc(void* out_ids, const void* logits, int rows, int vocab, int ld,
//                         int logits_are_f32, long long id_offset, void* out_values,
//                         cudaStream_t stream);
//
//   out_ids     int64 [rows]            winning index per row, plus id_offset
//   logits      fp32 or bf16 [rows, ld] (first `vocab` entries of each row are used)
//   out_values  fp32 [rows] or NULL     winning logit per row
//
// Same result as sl_argmax (ties to the lower index, a row of NaN / -inf yields index 0).
//
// Limits and rules
//   * rows <= SL_ARGMAX_NOALLOC_MAX_ROWS (256).  Larger requests are refused with
//     SL_NOALLOC_E_TOO_LARGE and a message on stderr; nothing is launched.
//   * The scratch is a file-scope __device__ array of SL_ARGMAX_NOALLOC_MAX_ROWS * 64 partial
//     (value, index) pairs = 128 KiB.  Every GPU that loads the library holds it until the
//     process exits.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) with that device current.  Make that first call outside any
//     stream capture; later calls only launch kernels.  The address is kept in a plain per-device table:
//     let one host thread make the first call on a device before several host threads call concurrently
//     (two racing first calls would both store the same address, but the store is not synchronised).
//   * All calls share the one array, which keeps whatever the previous call left in it; each
//     call overwrites every partial it later reads, so nothing needs clearing.  Two calls that
//     overlap on the GPU (different streams, no dependency) race on the array: serialise them.
//   * No cudaMalloc / cudaFree / allocating library routine is called, here or in the kernels.
//
// Return value: 0 on success, a positive cudaError_t from the runtime, or one of the negative
// codes below.
#pragma once

#include <cuda_runtime.h>

#define SL_ARGMAX_NOALLOC_MAX_ROWS 256
#define SL_NOALLOC_E_TOO_LARGE (-22)   /* rows beyond SL_ARGMAX_NOALLOC_MAX_ROWS */
#define SL_NOALLOC_E_BAD_ARG (-23)     /* null pointer, non-positive vocab, ld < vocab */
#define SL_NOALLOC_E_SETUP (-24)       /* the scratch symbol could not be resolved on this device */

#ifdef __cplusplus
extern "C" {
#endif
int sl_argmax_noalloc(void* out_ids, const void* logits, int rows, int vocab, int ld, int logits_are_f32,
                      long long id_offset, void* out_values, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
