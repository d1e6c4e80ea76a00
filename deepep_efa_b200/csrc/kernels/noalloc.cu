// Allocation-free variant of get_dispatch_layout: same kernel (layout.cu), scratch taken from a fixed
// array inside the library image instead of from an allocator. See noalloc.h for who needs this and for
// the rules. This entry point has no counterpart in the reference library.
#include "noalloc.h"

#include <cstdio>
#include <mutex>

#include "api.h"

namespace {

// Partial histograms + the completion ticket of the layout kernel. Lives in every GPU that loads this
// library. The NAME below is only a host-side handle: host code must never pass it to a kernel; the
// device address is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) int g_layout_scratch[DX_NOALLOC_MAX_SCRATCH_INTS];

constexpr int kMaxDevices = 64;
int* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_mu;
thread_local char g_last_error[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0) {
    std::snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
    return code;
}

// Device address of the scratch array on the CURRENT device (looked up on first use).
int* scratch_for_current_device(int* code) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        *code = fail(DX_NOALLOC_CUDA_ERROR, "cudaGetDevice failed or device index out of range (%lld)", dev);
        return nullptr;
    }
    std::lock_guard<std::mutex> g(g_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_layout_scratch);
        if (e != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            *code = fail(DX_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress failed on device %lld (error %lld)", dev, (long long)e);
            return nullptr;
        }
        g_scratch_ptr[dev] = static_cast<int*>(p);
    }
    return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int dx_get_dispatch_layout_noalloc(const int64_t* topk_idx, int num_tokens, int num_topk, int num_experts, int num_ranks,
                                              int* num_tokens_per_rank, int* num_tokens_per_expert, bool* is_token_in_rank,
                                              cudaStream_t stream) {
    g_last_error[0] = '\0';
    if (topk_idx == nullptr || num_tokens_per_rank == nullptr || num_tokens_per_expert == nullptr || is_token_in_rank == nullptr)
        return fail(DX_NOALLOC_BAD_ARGUMENT, "null pointer argument");
    if (num_tokens < 0 || num_topk < 1 || num_experts < 1 || num_ranks < 1 || num_ranks > dx::kMaxRanks || num_experts % num_ranks != 0)
        return fail(DX_NOALLOC_BAD_ARGUMENT, "need num_topk >= 1, 1 <= num_ranks <= 8 and num_experts a positive multiple of num_ranks");
    const size_t need = dx::layout_scratch_ints(num_experts, num_ranks, num_tokens);
    if (need > (size_t)DX_NOALLOC_MAX_SCRATCH_INTS)
        return fail(DX_NOALLOC_TOO_LARGE,
                    "problem needs %lld scratch ints but the built-in scratch holds %lld; use the allocating get_dispatch_layout",
                    (long long)need, (long long)DX_NOALLOC_MAX_SCRATCH_INTS);
    // same bound as the launcher's shared-memory request (experts + 2 * ranks bins), checked before anything is queued
    if ((size_t)(num_experts + 2 * num_ranks) * sizeof(int) > 48 * 1024)
        return fail(DX_NOALLOC_TOO_LARGE, "num_experts + 2 * num_ranks = %lld bins do not fit the kernel's shared-memory histogram",
                    num_experts + 2 * num_ranks);
    // With 8 ranks the kernel writes one token's eight membership bytes as a single 8-byte store; a bool* is only
    // guaranteed 1-byte alignment (a slice of a larger buffer), so an unaligned output is refused here instead of
    // faulting on the device.
    if (num_ranks == 8 && (reinterpret_cast<uintptr_t>(is_token_in_rank) & 7u) != 0)
        return fail(DX_NOALLOC_BAD_ARGUMENT, "with 8 ranks is_token_in_rank must be 8-byte aligned");
    if ((reinterpret_cast<uintptr_t>(topk_idx) & 7u) != 0 || (reinterpret_cast<uintptr_t>(num_tokens_per_rank) & 3u) != 0 ||
        (reinterpret_cast<uintptr_t>(num_tokens_per_expert) & 3u) != 0)
        return fail(DX_NOALLOC_BAD_ARGUMENT, "topk_idx must be 8-byte aligned and the count outputs 4-byte aligned");
    int code = DX_NOALLOC_OK;
    int* scratch = scratch_for_current_device(&code);
    if (scratch == nullptr) return code;
    // The array keeps whatever the previous call left. Only the completion ticket (first int) must be zero
    // when the kernel starts; the partial histograms are fully rewritten before they are read.
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int), stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DX_NOALLOC_CUDA_ERROR, "cudaMemsetAsync failed (error %lld)", (long long)e);
    }
    dx::LayoutArgs a{};
    a.topk_idx = topk_idx;
    a.num_tokens = num_tokens;
    a.num_topk = num_topk;
    a.num_experts = num_experts;
    a.num_ranks = num_ranks;
    a.num_tokens_per_rank = num_tokens_per_rank;
    a.num_tokens_per_expert = num_tokens_per_expert;
    a.is_token_in_rank = is_token_in_rank;
    a.scratch = scratch;
    e = dx::launch_layout(a, stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DX_NOALLOC_CUDA_ERROR, "kernel launch failed (error %lld)", (long long)e);
    }
    return DX_NOALLOC_OK;
}

extern "C" const char* dx_noalloc_last_error(void) { return g_last_error; }
