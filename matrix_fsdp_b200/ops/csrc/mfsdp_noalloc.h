// Allocation-free entry point of the kernel library.  It has no counterpart in the reference
// project (which ships no RMSNorm kernel and no C entry points at all); it exists for callers of
// this library that are not able to allocate device memory themselves.
//
// Who that is: code that drives these kernels from a context where cudaMalloc (or a framework's
// caching allocator) must not be reached -- for example a host thread that runs while another
// component owns the allocator lock, a plugin loaded into a process whose memory budget is fixed at
// start-up, or a C caller that links only this shared object and has no allocator of its own.  The
// regular mfsdp_rmsnorm_bwd() needs a caller-provided fp32 scratch matrix for the per-CTA partial
// sums of the weight gradient; this variant keeps that scratch inside the library instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the built-in scratch can serve and the number of partial rows it holds.
#define MFSDP_NOALLOC_MAX_HIDDEN 8192
#define MFSDP_NOALLOC_SCRATCH_ROWS 148

// RMSNorm backward without any allocation.
//
//   dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) [+ dres]        (bf16, [rows, H])
//   dw = (accumulate_dw ? dw : 0) + sum over rows of dy * xhat   (bf16, [H])
//
// Inputs dy, x ([rows, H] bf16), w ([H] bf16), rstd ([rows] fp32), optional dres ([rows, H] bf16) and
// outputs dx, dw are the caller's buffers.  The fp32 partial sums live in a fixed device array of
// MFSDP_NOALLOC_SCRATCH_ROWS x MFSDP_NOALLOC_MAX_HIDDEN floats (about 4.6 MiB) that is part of this
// library's image: every GPU that loads the library holds that array until the process exits.
//
// Returns 0 on success, -2 when H is not a multiple of 8 or exceeds MFSDP_NOALLOC_MAX_HIDDEN (or rows
// <= 0), otherwise the CUDA error code.  Calls no cudaMalloc / cudaFree and no allocating library
// routine.
//
// The first call on each device looks up the device address of the scratch array (a host-side query,
// no allocation); make that first call before starting any stream capture on that device.
//
// All calls on a device share the one scratch array.  It needs no clearing (each call overwrites
// every element it later reads), but two calls whose kernels overlap on the GPU -- different streams
// without ordering between them -- race on it: serialise them on one stream or with events.
int mfsdp_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                              const void* dres, void* dx, void* dw, int accumulate_dw, long long rows,
                              int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
