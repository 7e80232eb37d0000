// pk_gqa_decode_static: split-context GQA decode that performs no allocation at all.
//
// This entry point has no counterpart in the reference implementation.
//
// Who needs it: callers that must not allocate device memory at the point where they run
// attention. Examples: a host that has handed the whole device to another allocator and
// cannot ask it from this thread (a real-time audio/robotics loop, a plugin inside someone
// else's process); code running while an allocator lock is held; a fallback path entered
// after an out-of-memory error. pk_gqa_decode() asks such a caller to provide the
// [M, Hq, nsplit, head_dim + 2] float scratch itself; this variant keeps that scratch in a
// fixed array that is part of the loaded library image, so the call needs nothing but its
// inputs and outputs.
//
// Contract
//  * Arguments are those of pk_gqa_decode() without `ws`; results are identical.
//  * Limit: M * Hq * nsplit * (head_dim + 2) <= PK_GQA_STATIC_WS_FLOATS (2.03 MiB of floats;
//    e.g. 8 rows x 64 heads x 8 splits at head_dim 128). Larger problems are rejected with
//    PK_ERR_BAD_ARG before anything is launched; pk_gqa_decode_static_error() then returns a
//    sentence with the requested and the available size.
//  * Set-up: the first call on each device (with that device current) looks up the device
//    address of the array, which can also make the CUDA runtime load the module. Make that
//    first call during initialisation, before any stream capture starts on that device. Later
//    calls on the same device do no set-up.
//  * No cudaMalloc / cudaFree / allocating library call is made on any call, first or later.
//  * The array is shared by every call on a device. Nothing in it has to start at zero: the
//    split kernel writes every slot that the merge kernel reads. Two calls whose execution can
//    overlap (different streams, or different host threads on different streams) race on the
//    scratch; order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>

#define PK_GQA_STATIC_WS_FLOATS (8 * 64 * 8 * 130)

#ifdef __cplusplus
extern "C" {
#endif

int pk_gqa_decode_static(const void* q, const void* kcache, const void* vcache, const int* pos, int M, int Hq,
                         int Hkv, int head_dim, int ctx_cap, float scale, int nsplit, int window, int sink,
                         const void* gate_proj, int ld, void* out, cudaStream_t stream);

// Message of the last rejected call on the calling thread ("" if none).
const char* pk_gqa_decode_static_error(void);

#ifdef __cplusplus
}
#endif
