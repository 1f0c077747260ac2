// Allocation-free entry point of libprimus_b200.
//
// This entry point has no counterpart in the reference framework.  It exists for callers that must
// not allocate device memory at the point of the call: code running inside a memory-planned region
// (a fixed arena handed out once at start-up), plugins loaded into a host application that owns all
// cudaMalloc traffic, or latency-critical loops where an allocator call (and the implicit
// synchronisation a cudaMalloc / cudaFree may cause) is not acceptable.
//
// pb_rmsnorm_bwd_noalloc computes exactly what pb_rmsnorm_bwd computes (RMSNorm backward: the input
// gradient, optionally summed with a residual-stream gradient, and the weight gradient), but the fp32
// scratch that holds the per-CTA partial weight gradients is a fixed array inside the library's device
// image instead of a buffer supplied by the caller.  Inputs and outputs are still caller-owned.
//
// Limits and rules
//  * H (row width) <= PB_NOALLOC_MAX_H (8192), H % 8 == 0, row pitches % 8 == 0.  Up to 2^31 - 1 rows (more are
//    rejected with PB_NOALLOC_ERR_BAD_ARG).
//    Larger H is rejected with PB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//  * The scratch is PB_NOALLOC_MAX_PARTIALS x PB_NOALLOC_MAX_H floats = 296 x 8192 x 4 B = 9.25 MiB.  It is
//    part of the loaded library: every GPU on which the library is used holds that much memory until the
//    process exits.
//  * The first call on a device resolves the device address of the scratch (cudaGetSymbolAddress with
//    that device current) and remembers it; make that first call outside of any stream capture.
//  * The call itself uses no cudaMalloc, cudaFree or other allocating routine.
//  * All calls share the one scratch array and it keeps the previous call's contents.  Every call
//    overwrites the part it reads before reading it, so nothing needs clearing between calls; but two
//    calls that may overlap on the GPU (different streams, or different host threads without ordering)
//    race on it.  Serialise them on one stream or with events.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB_NOALLOC_MAX_H 8192
#define PB_NOALLOC_MAX_PARTIALS 296
#define PB_NOALLOC_ERR_TOO_LARGE (-10)
#define PB_NOALLOC_ERR_BAD_ARG (-2)

// dy, x, dres (may be NULL), dx: bf16 [rows, H] with row pitches lddy (dy) and ldx (x, dres, dx) in elements;
// w: bf16 [H]; rstd: fp32 [rows]; dw: fp32 [H] (dw_accumulate != 0: dw += result).
// Returns 0 on success, PB_NOALLOC_ERR_* or a cudaError_t value otherwise.
int pb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                           void* dx, float* dw, long rows, int H, long ldx, long lddy, int dw_accumulate,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
