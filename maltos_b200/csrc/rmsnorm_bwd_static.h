// RMSNorm backward that allocates nothing. This entry point has no counterpart in the reference framework: it exists
// for callers that cannot allocate device memory around the call - a C/C++ host that drives the library without the
// PyTorch caching allocator, or a region of a program in which cudaMalloc/cudaFree (which synchronise the device and
// may fail under memory pressure) are not acceptable. The regular entry point `mb_rmsnorm_bwd` takes its fp32
// partial-sum scratch from the caller; this one owns it as a file-scope array in device memory.
//
// Limits: hidden size H a multiple of 8 and at most MB_RMSNORM_STATIC_MAX_H; the scratch holds
// MB_RMSNORM_STATIC_MAX_BLOCKS x MB_RMSNORM_STATIC_MAX_H floats (9.5 MiB per device). A larger problem is rejected
// with a negative return code and a message in mb_last_error(); nothing is launched then.
//
// Set-up: the first call on each device resolves the address of the array (cudaGetSymbolAddress, which may initialise
// the module on that device). Make that first call outside any stream capture.
//
// Sharing: there is ONE scratch array per device. Two calls that may run at the same time on one device (different
// streams, or different host threads on different streams) race on it; issue them on one stream or order them with
// events. Calls on the same stream are safe back to back. Nothing in the scratch has to start at zero: every launch
// overwrites each partial row it later reads.
#pragma once
#include <cuda_runtime.h>

#define MB_RMSNORM_STATIC_MAX_H 8192
#define MB_RMSNORM_STATIC_MAX_BLOCKS 304

#ifdef __cplusplus
extern "C" {
#endif

// dx = d(RMSNorm)/dh applied to dy (+ dres when given); dw (bf16 and/or fp32, optionally accumulated) = sum over rows of
// dy * normalised(h). Same arguments and results as mb_rmsnorm_bwd minus the scratch pointer. Returns 0 on success,
// a cudaError_t value for a CUDA failure, or < 0: -1 bad H, -2 problem larger than the static scratch.
int mb_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dx,
                          void* dw_bf16, float* dw_f32, int accumulate_dw, long long rows, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
