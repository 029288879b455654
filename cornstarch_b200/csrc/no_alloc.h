// Column-sum entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project: it exists for users of this library
// whose code runs where cudaMalloc is off limits, for example inside a framework's allocator callback,
// in a real-time inference loop that has frozen its memory pool, or in a host process that shares the
// GPU under a fixed memory budget and may not grow its footprint after start-up.  Such callers still
// own the input and output buffers; what they cannot provide is the temporary per-block partial-sum
// buffer that csb_colsum needs.  Here that buffer lives inside the library as a fixed, file-scope
// device array.
//
//   out[c] (+)= sum over rows of x[r][c]        x: bf16 [rows][H] row-major, out: fp32 or bf16 [H]
//
// Limits: H must be a multiple of 8 and at most CSB_COLSUM_NOALLOC_MAX_H; any number of rows.  x must be
// 16-byte aligned (it is read in 16-byte pieces; with H a multiple of 8 every row then is), out aligned
// to its element size.  A misaligned pointer is refused with CSB_ERR_BAD_ARG (-1); nothing is launched.
// Larger H is refused with CSB_ERR_TOO_LARGE (-4) and a message on stderr; nothing is launched.
//
// Things to know before using it:
//   * Every GPU that loads the library carries the scratch array (about 9.3 MiB) until the process ends.
//   * The first call on each device looks up the device address of the array.  Make that first call
//     outside any CUDA stream capture, with the device you mean to use current.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in it.
//     The kernels overwrite every slot they later read, so stale contents are harmless, but two calls
//     that overlap on the GPU (different streams, no ordering between them) race on the array.
//     Order such calls with events or issue them on one stream.
//   * Neither this function nor anything it calls uses cudaMalloc, cudaFree or an allocating library routine.
#pragma once

#define CSB_COLSUM_NOALLOC_MAX_H 8192
#define CSB_COLSUM_NOALLOC_MAX_PARTS 296

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, a negative CSB_ERR_* code when the arguments are refused, or a cudaError value.
int csb_colsum_noalloc(const void* x, void* out, int out_fp32, int accumulate, int rows, int H, void* stream);

#ifdef __cplusplus
}
#endif
