// Allocation-free entry point of the kernel library.
//
// This declaration has no counterpart in the reference project: it exists for callers of
// this library that are not able to obtain device memory themselves. Examples are code that
// runs while a memory pool is frozen (inside an allocator callback, or in a process whose
// whole device budget was handed to another framework up front), plug-ins that are only
// given input and output buffers by their host application, and real-time loops where a call
// into the CUDA allocator is an unbounded stall. Such callers still pass their inputs and
// outputs; the scratch space that the regular entry point asks the caller to provide lives
// inside the library instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch area (see tdllm_rmsnorm_bwd_noalloc).
#define TDLLM_NOALLOC_MAX_HIDDEN 4096
#define TDLLM_NOALLOC_PARTS 256
// bytes of device memory every GPU that loads the library holds until the process exits
#define TDLLM_NOALLOC_SCRATCH_BYTES (TDLLM_NOALLOC_PARTS * TDLLM_NOALLOC_MAX_HIDDEN * 4)

// RMSNorm backward without any allocation. Same mathematics and arguments as
// tdllm_rmsnorm_bwd, minus the scratch pointer: the per-block partial sums of the weight
// gradient go to a fixed 4 MiB array inside the library.
//
//  * H must be a multiple of 8 and at most TDLLM_NOALLOC_MAX_HIDDEN; larger sizes are rejected
//    with a non-zero return code and a message in tdllm_last_error().
//  * The first call on each device looks up the array's device address (once per device, with
//    that device current). Make that first call before starting any stream capture, and make it from one
//    thread: the per-device cache is filled without a lock (concurrent first calls would store the same
//    value, which is harmless, but is not something this header promises).
//  * The function calls no cudaMalloc / cudaFree and no allocating library routine.
//  * Every call on a device shares the one array. Each call overwrites all partial sums it later
//    reads, so nothing needs clearing between calls, but two calls that overlap on the GPU
//    (different streams, no ordering between them) race on it: serialise them.
int tdllm_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd,
                              const void* dres_in, void* dx, void* dw, int dw_fp32,
                              int dw_accumulate, int rows, int H, void* stream);

#ifdef __cplusplus
}
#endif
