// Entry points that never allocate.
//
// ptb_rmsnorm_bwd_static has no counterpart in the reference framework: it is an addition of this library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the static variant can use: n_ctas * H fp32 values (4 MiB).
#define PTB_RMS_STATIC_SCRATCH_FLOATS (1 << 20)

// RMSNorm backward, same arguments and results as ptb_rmsnorm_bwd minus the caller-provided `dw_partial`
// scratch: the per-CTA partial sums of dw go to a fixed device array that is part of the library image.
//
// For callers that cannot allocate device memory at the point of the call: a host program that links
// the library without a tensor allocator behind it, or a step loop that has handed all free device
// memory to its own pools and where a cudaMalloc would fail or stall every stream of the device.
// The function calls no allocator of any kind (no cudaMalloc / cudaFree, no library routine that
// allocates): it launches two kernels on `st` and returns.
//
// * The first call on each device looks up the address of the scratch array (cudaGetSymbolAddress);
//   make that first call before any stream capture begins.
// * n_ctas * H must not exceed PTB_RMS_STATIC_SCRATCH_FLOATS; larger requests are rejected with -1 and a
//   message in ptb_last_error(), nothing is launched.
// * All calls on one device share the one array.  Every launch overwrites the part it reads back, so
//   nothing has to start at zero; but two calls that overlap in time (different streams, or different
//   host threads on different streams) race on it.  Issue them on one stream, or order them with events.
int ptb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, int n_ctas,
                           long long rows, int H, const void* dresid, int bf16, cudaStream_t st);

#ifdef __cplusplus
}
#endif
