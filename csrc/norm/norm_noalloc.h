// LayerNorm / RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this
// library whose process must not call cudaMalloc at the time they need the op: a serving
// or real-time loop that carved up all device memory at start-up and treats any later
// allocation as a fault, a host application that embeds the library under an allocator it
// does not control, or code running at a point where an allocation's implicit device
// synchronisation is not acceptable.
//
// st_norm_bwd needs an fp32 scratch buffer from its caller.  st_norm_bwd_noalloc computes
// exactly the same result but keeps that scratch in a fixed array inside the library
// (ST_NORM_BWD_NOALLOC_MAX_ELEMS floats = 4.6 MiB, reserved on every GPU that loads the
// library until the process exits).  It never calls cudaMalloc, cudaFree or any other
// allocating routine.
//
//   * Limit: 2 * ctas(rows) * d must not exceed ST_NORM_BWD_NOALLOC_MAX_ELEMS, where
//     ctas(rows) = min(rows, 2 * number of SMs).  On a 148-SM B200 that covers every row
//     count for d <= 2048, and d up to 8192 for rows <= 74.  Larger problems are rejected
//     with ST_ERR_TOO_LARGE and a message in st_last_error(); nothing is launched.
//   * The first call on each device looks up the device address of the array (the device
//     must be current).  Make that first call before starting any stream capture.
//   * "Allocates nothing" is true once the array exists.  The CUDA runtime loads a module's
//     device variables lazily, so the 4.6 MiB array may only be materialised by the first norm
//     kernel or the first call of this entry point on a device.  A process that hands out all
//     device memory itself should therefore make one warm-up call per device (or any other norm
//     call of this library) at start-up, BEFORE it carves up the memory; otherwise that first call
//     can be the one that fails for lack of memory.
//   * Host threads: the cached address is written without a lock.  Concurrent first calls from
//     several threads on one device all store the same value, which is harmless, but the simplest
//     rule is to make the per-device warm-up call from one thread before the others start.
//   * Every call shares the one array.  Each call overwrites the part of it that it later
//     reads, so no clearing is needed between calls, but two calls that overlap on the GPU
//     (different streams) race on it: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ST_NORM_BWD_NOALLOC_MAX_ELEMS (2 * 296 * 2048)

// Same arguments and semantics as st_norm_bwd without the scratch pointer.  Returns 0 on
// success; ST_ERR_TOO_LARGE (3) when the problem exceeds the fixed scratch capacity.
int st_norm_bwd_noalloc(int rms, const void* dy, const void* x, const void* gamma,
                        const float* mean, const float* rstd, const void* dres, void* dx,
                        float* dgamma, float* dbeta, int accumulate, int rows, int d,
                        void* stream);

#ifdef __cplusplus
}
#endif
