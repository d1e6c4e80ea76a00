// Allocation-free entry point for the dispatch-layout computation.
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: code that must compute a dispatch layout from a place where device memory cannot be
// requested — a plugin or a foreign-language runtime that was handed raw device pointers and owns no
// allocator, a real-time serving loop that forbids cudaMalloc after start-up because it synchronises the
// whole device, or a host whose memory pool is fully reserved by another framework. The regular path
// (get_dispatch_layout in the Python module) creates its outputs and its scratch buffer through the
// PyTorch allocator; this one takes caller-owned outputs and keeps its scratch in a fixed array that is
// part of the loaded library image.
//
// Limits and rules:
//  * The scratch array holds DX_NOALLOC_MAX_SCRATCH_INTS ints (about 1 MiB) on every GPU that loads the
//    library, until the process exits. A call needs 1 + ceil(T / 256) * (E + R) ints; larger problems are
//    rejected with DX_NOALLOC_TOO_LARGE and nothing is launched.
//  * The first call on each device looks up the device address of the array (with that device current).
//    Make that first call before starting any stream capture.
//  * All calls on a device share the one array. Two calls whose kernels overlap on the GPU (different
//    streams, no dependency) race on it; serialise them on one stream or with events.
//  * `stream` must belong to the device that is current when the call is made (the scratch address is the current
//    device's copy of the array).
//  * With num_ranks == 8 `is_token_in_rank` must be 8-byte aligned (each token's row is written with one store);
//    an unaligned pointer is refused with DX_NOALLOC_BAD_ARGUMENT and nothing is launched.
//  * Nothing is allocated or freed: no cudaMalloc/cudaFree, no PyTorch tensors.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define DX_NOALLOC_MAX_SCRATCH_INTS (1 + 256 * 1032)

#define DX_NOALLOC_OK 0
#define DX_NOALLOC_BAD_ARGUMENT (-1)
#define DX_NOALLOC_TOO_LARGE (-2)
#define DX_NOALLOC_CUDA_ERROR (-3)

#ifdef __cplusplus
extern "C" {
#endif

// topk_idx          [num_tokens, num_topk] int64 on the current device, -1 = no selection
// num_tokens_per_rank   [num_ranks]   int32 out
// num_tokens_per_expert [num_experts] int32 out
// is_token_in_rank      [num_tokens, num_ranks] bool (1 byte each) out
// Returns DX_NOALLOC_OK or one of the negative codes above; dx_noalloc_last_error() describes the failure.
__attribute__((visibility("default"))) int dx_get_dispatch_layout_noalloc(const int64_t* topk_idx, int num_tokens, int num_topk,
                                                                          int num_experts, int num_ranks, int* num_tokens_per_rank,
                                                                          int* num_tokens_per_expert, bool* is_token_in_rank,
                                                                          cudaStream_t stream);

// Message of the last failure on the calling thread (empty string if none).
__attribute__((visibility("default"))) const char* dx_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
