// BatchNorm backward without any memory allocation on the call path.
//
// This entry point has no counterpart in the reference (keras-team/keras has no C ABI and leaves
// all temporaries to its backend's allocator).  It exists for callers of libkb200.so that are not
// allowed to allocate: a C or C++ serving/runtime process that links the library without torch
// (so there is no caching allocator to hand out the 5*C-float temporary), and processes that have
// already handed all free HBM to their own pools, where cudaMalloc can fail and, like cudaFree,
// stalls every stream of the device while it runs.
//
// The temporary that kb200_bn_bwd_reduce / kb200_bn_bwd_apply take from the caller (2*C sums and
// 3*C coefficients, fp32) lives in a file-scope `static __device__` array of
// KB200_BN_STATIC_MAX_C * 5 floats (80 KiB) instead.  The host asks for its address once per
// device (cudaGetSymbolAddress, with that device current) and hands the pointer to the kernels.
//
// Rules for callers
//  * C must be <= KB200_BN_STATIC_MAX_C (and a multiple of 8 for bf16, 4 for fp32); larger C is
//    refused with a non-zero return and a message in kb200_last_error(); nothing is launched.
//  * The first call on a device performs the address look-up.  Call kb200_bn_bwd_static_setup()
//    (or make one ordinary call) on every device at start-up, before any stream capture begins,
//    so that later calls only enqueue work on `stream`.
//  * Every call on a device shares the one array.  The first 2*C floats must be zero when the
//    reduction starts; the call clears them itself on `stream` (cudaMemsetAsync), so callers need
//    not.  The remaining 3*C floats are fully written before they are read.  Stale values beyond
//    5*C from an earlier, wider call are never read.
//  * Two calls that can run at the same time on one device (different streams with no ordering
//    between them, or two host threads) race on the array and give wrong gradients.  Order them
//    on one stream or with events.
#pragma once
#include <cuda_runtime.h>

#define KB200_BN_STATIC_MAX_C 4096

#ifdef __cplusplus
extern "C" {
#endif

// Look up the scratch address for the current device.  Returns 0 on success.
int kb200_bn_bwd_static_setup(void);

// dx = d(loss)/dx, dres = dy masked by (y > 0) (may be null), dgamma/dbeta fp32[C] (dgamma may be
// null).  dy, x, y (y may be null: no ReLU mask), dx, dres are [M, C] of `dtype` (0 = fp32,
// 1 = bf16); mean, invstd, gamma (may be null) are fp32[C].  Returns 0 on success.
int kb200_bn_bwd_static(const void* dy, const void* x, const void* y, const float* mean, const float* invstd, const float* gamma, void* dx,
                        void* dres, float* dgamma, float* dbeta, long long M, int C, int dtype, cudaStream_t stream);

// Capacity of the static scratch in channels (KB200_BN_STATIC_MAX_C).
int kb200_bn_bwd_static_max_channels(void);

#ifdef __cplusplus
}
#endif
