// Entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference project; it exists for users of this library
// who run inside a memory pool they do not own -- an inference server or a training
// runtime that has handed every byte of the GPU to its own allocator, or a plugin that is
// called while that allocator is locked.  Such callers cannot call cudaMalloc (nor any
// library routine that might), yet the regular RMSNorm backward needs scratch space for
// its per-block partial sums of the weight gradient.
//
// ftb200_rmsnorm_bwd_noalloc computes exactly what ftb200_rmsnorm_bwd computes, but keeps
// the partial sums in an array that is part of the library image itself (a file-scope
// __device__ array of FTB200_NOALLOC_SCRATCH_FLOATS floats, about 9.3 MiB, resident on
// every GPU that loads the library until the process exits).  The caller passes only its
// inputs and outputs.
//
//  * Sizes: D must be a multiple of 8 and at most 8192, and (2 * SM count) * D must not
//    exceed FTB200_NOALLOC_SCRATCH_FLOATS; anything larger is refused with
//    FTB200_E_TOOBIG (-4) before anything is launched.
//  * First call on a device: looks up the device address of the array once
//    (cudaGetSymbolAddress with that device current) and remembers it.  Make that first
//    call outside of any stream capture.  Host threads may race on that first call: the
//    remembered address is an atomic, and every thread resolves the same value.
//  * No cudaMalloc, cudaFree or allocating library call is made, on any call.
//  * All calls share the one array.  Every call overwrites the part it uses before reading
//    it, so nothing has to be cleared between calls; but two calls that overlap on the same
//    GPU (different streams) race on it -- serialise them.
#pragma once

#include <cuda_runtime.h>

#define FTB200_NOALLOC_SCRATCH_FLOATS (296 * 8192)

#ifdef __cplusplus
extern "C" {
#endif

// dy, x, dres (may be null), dx: [T, D] bf16; w, dw: [D] bf16; rstd: [T] fp32.
// dx = dres + d(rmsnorm)/dx, dw (+)= d(rmsnorm)/dw.  Returns 0 or a negative FTB200_E_* code.
int ftb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, void* dw, int T, int D, int accumulate_dw, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
