// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a host that has handed all
// device memory to its own pool at start-up and forbids further driver allocations, a real-time
// or serving loop that may not take the allocator's locks or its implicit synchronisation, or a
// plugin loaded into a process whose allocator it does not own.  The regular entry point
// (ws_rmsnorm_bwd) needs a caller-provided scratch buffer for the per-block partial sums of the
// weight gradient, which in practice means one more allocation per call; this one brings its
// own.
//
// How: the partial sums live in an array that is part of the library image itself (a file-scope
// device array of WS_STATIC_SCRATCH_FLOATS floats, about 3.5 MiB).  Every GPU that loads the
// library holds that memory until the process exits, whether or not this function is ever
// called.  The function itself calls no cudaMalloc, no cudaFree and no allocating library
// routine; inputs and outputs are the caller's.
//
// Set-up: the first call on each device looks up the device address of the array (one
// cudaGetSymbolAddress with that device current) and caches it.  Make that first call during
// initialisation, before any stream capture begins, with the device you will use current.
//
// Limits and sharing:
//   * d must be a multiple of 128 and at most 2048: that is the limit that binds.  A wider row is
//     rejected with WS_STATIC_ERR_BAD_SHAPE before any work is launched (ws_static_scratch_strerror
//     gives the text).  The number of rows is free: the kernel never uses more than 444 partial
//     rows (three blocks on each of 148 SMs) however many rows there are, and the array holds
//     exactly 444 rows of 2048 floats.  WS_STATIC_ERR_TOO_LARGE guards the array bound itself and
//     cannot be returned while the width limit stands.
//   * All calls on a device share the one array, and it keeps whatever the previous call left
//     in it.  Each call overwrites every element it later reads, so nothing has to be cleared,
//     but two calls that overlap in time on the same GPU (different streams, or different
//     threads) race on it and both results are garbage.  Serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WS_STATIC_SCRATCH_FLOATS (444 * 2048)

#define WS_STATIC_ERR_BAD_SHAPE (-1)
#define WS_STATIC_ERR_LAUNCH (-2)
#define WS_STATIC_ERR_TOO_LARGE (-30)
#define WS_STATIC_ERR_SYMBOL (-31)

// Same contract as ws_rmsnorm_bwd followed by the column-sum reduction:
//   dx_out  = (dres + rmsnorm_backward(dz; x, rstd, w)) * (1 + out_scale)      [rows, d]
//   dx_bf16 = BF16 copy of dx_out (may be NULL)
//   dw_out  = sum over rows of dz * x_hat                                       [d], FP32
// x, dres and dx_out are FP32 when x_bf16 == 0, BF16 otherwise; dz is BF16; dres and out_scale
// may be NULL.  Returns 0 or one of the WS_STATIC_ERR_* codes.
int ws_rmsnorm_bwd_static(const void* dz, const void* x, int x_bf16, const float* rstd, const float* w,
                          const void* dres, const float* out_scale, int rows, int d, void* dx_out,
                          void* dx_bf16, float* dw_out, cudaStream_t stream);

const char* ws_static_scratch_strerror(int code);

#ifdef __cplusplus
}
#endif
