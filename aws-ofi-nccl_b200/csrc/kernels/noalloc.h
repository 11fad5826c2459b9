// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference plugin; it exists for users of this library
// that run where device allocation is off limits: code executing inside another framework's
// memory-pool callback, inside a region where the allocator is locked, or in a plugin hook that
// NCCL invokes while it holds its own allocator state. Such callers cannot create the fp32 staging
// rows that the RMSNorm backward needs for its weight-gradient partial sums, so this variant keeps
// those rows in a fixed array that is part of the loaded library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the fixed staging area can serve.
#define B200_NOALLOC_MAX_H 8192      /* hidden size (elements per row), must also be a multiple of 8 */
#define B200_NOALLOC_MAX_ROWS 296    /* partial-sum rows = CTAs launched (2 per SM on a 148-SM part) */

// RMSNorm backward: dx = d(loss)/d(x) (+ dres), dw (+)= d(loss)/d(w), same maths and argument
// meaning as b200_rmsnorm_bwd, minus the caller-provided staging buffer.
//
//  * Allocates nothing: no cudaMalloc/cudaFree, no allocating library call. The staging rows
//    (B200_NOALLOC_MAX_ROWS x B200_NOALLOC_MAX_H floats, about 9.3 MiB) live in a file-scope
//    device array; every GPU that loads the library holds that memory until the process exits.
//  * The first call on a device looks up the array's device address (one cudaGetSymbolAddress with
//    that device current). Make that first call before starting any stream capture.
//  * The device must be current on the calling thread; the function does not switch devices.
//  * H above B200_NOALLOC_MAX_H (or not a multiple of 8) is refused with error 10004 / 10001; so is
//    any of dy, x, w, dres, dx, dw that is not 16-byte aligned (10001): rows move as 16-byte vectors.
//  * The looked-up address belongs to the device's context and is cached for the life of the
//    process; it does not survive a cudaDeviceReset.
//  * All calls share the one staging array, which keeps the previous call's contents. Every row a
//    call reads is fully rewritten by that call first, so nothing needs clearing — but two calls
//    that overlap in time on the same GPU (different streams) race on it. Serialise them.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, void* dw, int accumulate_dw, int T, int H, void* stream);

#ifdef __cplusplus
}
#endif
