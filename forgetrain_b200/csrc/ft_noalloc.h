// Entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine; it exists for users of this
// library who call the kernels from places where a device allocation is impossible or
// forbidden: code that runs while a stream is being captured into a CUDA graph (cudaMalloc is
// illegal there), runtimes that hand every byte of device memory to a pre-sized pool at start-up
// and treat any later allocation as a fault, and plain C / C++ hosts that have no tensor
// allocator to borrow scratch from.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size and row-partial count the built-in scratch can hold.
#define FT_NOALLOC_MAX_HIDDEN 8192
#define FT_NOALLOC_MAX_PARTIALS 148

// RMSNorm backward (same math as ft_rmsnorm_bwd) whose weight-gradient partial sums live in a
// scratch array compiled into the library (FT_NOALLOC_MAX_PARTIALS x FT_NOALLOC_MAX_HIDDEN
// floats = 4.6 MiB, held by every GPU that loads the library until the process exits) instead
// of a caller-provided buffer. The call performs no cudaMalloc / cudaFree and calls no
// allocating routine.
//
//   dy, h, w  : bf16 [T][H], [T][H], [H];   rstd : fp32 [T]
//   dres      : bf16 [T][H] or NULL (added to the result)
//   dx_out    : bf16 [T][H] (may alias dres)
//   dw        : fp32 [H], overwritten (accumulate == 0) or added to (accumulate != 0)
//
// Returns 0 on success, -1 for an unsupported hidden size (the kernels exist for H = 256, 512,
// 1024, 2048, 4096 and 8192), -2 when H exceeds FT_NOALLOC_MAX_HIDDEN,
// -3 when the address of the scratch array could not be obtained, -100 for a launch error.
//
// The first call on each device looks up the device address of the scratch array (with that
// device current) and caches it; make that first call outside any stream capture. All calls
// on one device share the one array: two calls whose kernels overlap on the GPU (different
// streams without an ordering between them) race on it. Calls on one stream are safe; the
// kernels rewrite every scratch row they later read, so stale contents never leak in.
int ft_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const void* rstd,
                           const void* dres, void* dx_out, void* dw, int accumulate, int T, int H,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
