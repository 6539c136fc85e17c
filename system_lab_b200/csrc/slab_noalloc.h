// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference: it exists for callers that drive these kernels
// from places where device memory cannot be requested -- a serving loop or a plugin that was handed a
// fixed memory budget and must not grow it, a real-time thread where an allocator call (and the implicit
// device synchronisation a cudaMalloc/cudaFree may bring) is off limits, or host code that has no
// allocator of its own to borrow (no PyTorch caching allocator behind it).
//
// The regular RMSNorm backward (`slab_rmsnorm_bwd`) asks its caller for a scratch matrix in which every
// thread block leaves its partial sum of the gain gradient.  The variant below keeps that scratch inside
// the library instead, in a fixed device array that is part of the loaded module, so the caller passes
// only inputs and outputs.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the built-in scratch covers.  The array holds SLAB_NOALLOC_MAX_BLOCKS rows of
// SLAB_NOALLOC_MAX_H floats (296 x 8192 x 4 bytes = 9.25 MiB) plus a few dozen ticket counters; every GPU that
// loads the library keeps that much reserved until the process exits, whether or not this entry point is ever
// called.  The kernel sizes its grid so that its partial rows (one per thread block plus one per group of eight
// blocks) fit those SLAB_NOALLOC_MAX_BLOCKS rows; elementwise.cu checks the tie at compile time.
#define SLAB_NOALLOC_MAX_H 8192
#define SLAB_NOALLOC_MAX_BLOCKS 296

// Return codes besides CUDA error numbers (> 0) and 0 for success.
#define SLAB_NOALLOC_ERR_SHAPE (-100)      /* H is not a multiple of 8 */
#define SLAB_NOALLOC_ERR_TOO_LARGE (-101)  /* H exceeds SLAB_NOALLOC_MAX_H: use slab_rmsnorm_bwd with your own scratch */
#define SLAB_NOALLOC_ERR_DEVICE (-102)     /* device ordinal outside the table kept by the library */

// RMSNorm backward without any allocation.
//
//   dx[r, :] = rstd[r] * (g[r, :] * w) - x[r, :] * rstd[r]^3 * mean(g[r, :] * w * x[r, :])  (+ gres[r, :] if given)
//   dw[:]    = sum_r g[r, :] * x[r, :] * rstd[r]
//
// g, x, gres (optional, may be NULL), dx: bf16 [rows, H]; w, dw: bf16 [H]; rstd: fp32 [rows] as written by
// slab_rmsnorm_fwd.  All pointers are device pointers of the current device; work is enqueued on `stream`.
//
// * Nothing is allocated or freed, by this function or by anything it calls.
// * The first call on each device looks up the device address of the built-in scratch (one
//   cudaGetSymbolAddress with that device current) and remembers it.  Make that first call outside of any
//   stream capture, and not from two threads at once for the same device.
// * Every call on a device uses the same scratch.  Two calls whose kernels may run at the same time on one
//   GPU (different streams, or different processes' threads sharing this library instance) race on it and
//   give wrong dw; serialise them.  The partial rows need not start at zero -- each launch rewrites every row
//   it later reads -- so what the previous call left behind is harmless.  The ticket counters of the in-kernel
//   reduction start at zero when the library is loaded and every completed launch leaves them at zero.
// * rows <= 0 is valid: dx is not touched and dw is written as zeros, as slab_rmsnorm_bwd does.
// * H above SLAB_NOALLOC_MAX_H is refused with SLAB_NOALLOC_ERR_TOO_LARGE and a line on stderr; nothing is
//   launched in that case.
int slab_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, const void* gres,
                             void* dx, void* dw, int rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
