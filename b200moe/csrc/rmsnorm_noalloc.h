// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for
// code that sits where cudaMalloc is off limits: a region being recorded into a
// CUDA graph, a callback running on a stream, a plugin living inside somebody
// else's memory pool, or a real-time loop that may not touch the allocator.
// The regular entry point (b2_rmsnorm_bwd) needs a caller-provided fp32 scratch
// of [parts, D] for the per-block partial sums of the gain gradient; here that
// scratch is a fixed array inside the library image, so the caller passes only
// inputs and outputs.
//
// Limits and rules
//   * D must be a multiple of 8 and at most B2_NOALLOC_MAX_D (8192); rows >= 1.
//     Anything else is refused with a negative code before any launch; use
//     b2_rmsnorm_bwd_noalloc_strerror(code) for the text.
//   * The scratch is B2_NOALLOC_PARTS x B2_NOALLOC_MAX_D floats (148 x 8192 x 4 B
//     = 4.6 MiB).  Every GPU that loads the library holds that much until the
//     process exits.
//   * The first call on each device looks up the scratch's device address
//     (cudaGetSymbolAddress) with that device current.  Make that first call
//     before starting any stream capture on the device.
//   * All calls on one device share the one scratch array, which keeps whatever
//     the last call left in it.  Nothing in it has to start at zero: each call
//     overwrites every element it later reads.  Two calls that overlap on the
//     GPU (different streams, no ordering between them) race on it; order them.
//   * dy, x, dx and (when given) residual are dense row-major [rows, D] bf16 (row pitch exactly D elements) and
//     start on a 16-byte boundary: the kernels move eight bf16 per access.  w, rstd and dw are 4-byte aligned.
//     A pointer off that grid is refused with code -8 before any launch; it never reaches the device.
//   * dx may be the same buffer as residual (each element is read before it is written by the same thread).
//     dx must not alias dy or x.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once
#include <cuda_runtime.h>

#define B2_NOALLOC_PARTS 148
#define B2_NOALLOC_MAX_D 8192

#ifdef __cplusplus
extern "C" {
#endif

// dx[rows,D] (bf16) = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ residual if not null)
// dw[D] (fp32)      = sum over rows of dy * xhat          (overwritten)
// dy, x, residual, dx: bf16 [rows, D]; w: fp32 [D]; rstd: fp32 [rows].
// Returns 0, or a negative code (see b2_rmsnorm_bwd_noalloc_strerror).
int b2_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const void* residual,
                           void* dx, float* dw, int rows, int D, cudaStream_t stream);

const char* b2_rmsnorm_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
