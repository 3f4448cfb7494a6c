// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for programs that run with a
// fixed memory plan (a captured CUDA graph, a serving process whose pool is handed out at start-up, a
// host that forbids cudaMalloc after initialisation): the weight-gradient partial sums that the regular
// entry point `ttcd_rmsnorm_bwd` expects in a caller-provided buffer live here in an array that is part
// of the library image itself, so the call performs no cudaMalloc / cudaFree and calls no library that
// allocates.
//
// What the caller has to know
//  * Limits.  D (the normalised width) must be a multiple of 8 and at most TTCD_NO_ALLOC_MAX_D; larger D
//    is refused with TTCD_NO_ALLOC_ERR_TOO_LARGE and nothing is launched.  The array holds
//    TTCD_NO_ALLOC_MAX_BLOCKS x TTCD_NO_ALLOC_MAX_D floats (1.16 MiB) per device.  Any number of rows.
//  * First call.  The first call on each device looks up the array's device address once
//    (cudaGetSymbolAddress) and raises the kernel's dynamic shared-memory limit.  Make that first call
//    during start-up, before any stream capture begins; later calls only launch two kernels.
//  * Contents.  The array keeps whatever the previous call left in it.  Nothing in it has to be zero:
//    every call overwrites all the entries it later reads.
//  * Concurrency.  There is one array per device.  Two calls that may overlap on the same device (two
//    streams, two threads, two graphs replayed concurrently) race on it; order them on one stream or
//    with events.  Calls on different devices are independent.  The host-side table of looked-up addresses
//    is filled without a lock: two host threads that make the very first call on one device at the same
//    time both run the look-up and store the same value, which is harmless.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TTCD_NO_ALLOC_MAX_D 2048
#define TTCD_NO_ALLOC_MAX_BLOCKS 148

#define TTCD_NO_ALLOC_OK 0
#define TTCD_NO_ALLOC_ERR_SHAPE (-1)      /* null pointer, rows <= 0, D <= 0 or D not a multiple of 8 */
#define TTCD_NO_ALLOC_ERR_TOO_LARGE (-3)  /* D > TTCD_NO_ALLOC_MAX_D */
#define TTCD_NO_ALLOC_ERR_DEVICE (-5)     /* device ordinal out of range, or the address look-up failed */

// dx[rows][D]  = d/ds of  y = s * rstd * w  applied to dy  (+ dres when dres is not null)
// dw[D] (fp32) = sum over rows of dy * s * rstd
// dy, s, dres, dx: bf16 [rows][D] contiguous; w: bf16 [D] or null (then dw is not written and may be null);
// rstd: fp32 [rows] saved by the forward.  All pointers are device pointers on the current device.
// Returns one of the codes above, or a positive cudaError_t from the launches.
int ttcd_rmsnorm_bwd_no_alloc(const void* dy, const void* s, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw, long long rows, int D, void* stream);

#ifdef __cplusplus
}
#endif
