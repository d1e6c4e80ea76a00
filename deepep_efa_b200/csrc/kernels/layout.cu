// get_dispatch_layout: from topk_idx[T,K] compute how many tokens go to every rank and expert and the
// [T,R] membership matrix, in ONE launch that needs no pre-zeroed outputs.
//
// Each CTA histograms 256 tokens in shared memory, stores its partial histogram, takes a ticket, and
// the last CTA to finish sums the partials. Experts are block-partitioned over ranks:
// expert e lives on rank e / (E/R). A selection of -1 (or out of range) is ignored.
//
// Reference counterpart: csrc/kernels/layout.cu:9-149 (one CTA per 4 experts / 8 ranks, every CTA
// re-reading all of topk_idx). Outputs are identical: num_tokens_per_rank[R] i32,
// num_tokens_per_expert[E] i32, is_token_in_rank[T,R] bool.
#include "api.h"
#include "prims.cuh"

namespace dx {

constexpr int kLayoutThreads = 256;

size_t layout_scratch_ints(int num_experts, int num_ranks, int num_tokens) {
    const size_t ctas = (num_tokens + kLayoutThreads - 1) / kLayoutThreads;
    return 1 + (ctas > 0 ? ctas : 1) * (size_t)(num_experts + num_ranks);
}

__global__ void __launch_bounds__(kLayoutThreads) layout_kernel(const LayoutArgs a) {
    extern __shared__ int s_hist[];  // [E] experts then [R] ranks
    const int E = a.num_experts, R = a.num_ranks, K = a.num_topk;
    const int L = E / R;
    const int bins = E + R;
    for (int i = threadIdx.x; i < bins; i += kLayoutThreads) s_hist[i] = 0;
    __syncthreads();

    const int t = blockIdx.x * kLayoutThreads + threadIdx.x;
    uint32_t mask = 0;
    if (t < a.num_tokens) {
        const int64_t* row = a.topk_idx + (size_t)t * K;
        for (int k = 0; k < K; ++k) {
            const int64_t e = row[k];
            if (e >= 0 && e < E) {
                atomicAdd(&s_hist[(int)e], 1);
                mask |= 1u << ((int)e / L);
            }
        }
        if (R == 8) {
            uint64_t packed = 0;
#pragma unroll
            for (int r = 0; r < 8; ++r) packed |= (uint64_t)((mask >> r) & 1u) << (8 * r);
            *reinterpret_cast<uint64_t*>(a.is_token_in_rank + (size_t)t * 8) = packed;
        } else {
            for (int r = 0; r < R; ++r) a.is_token_in_rank[(size_t)t * R + r] = (mask >> r) & 1u;
        }
    }
    // per-rank counts: one ballot per rank, one shared atomic per warp
    for (int r = 0; r < R; ++r) {
        const unsigned b = __ballot_sync(0xffffffffu, (mask >> r) & 1u);
        if ((threadIdx.x & 31) == 0 && b) atomicAdd(&s_hist[E + r], __popc(b));
    }
    __syncthreads();

    int* partial = a.scratch + 1 + (size_t)blockIdx.x * bins;
    for (int i = threadIdx.x; i < bins; i += kLayoutThreads) partial[i] = s_hist[i];

    if (cta_is_last(a.scratch, gridDim.x)) {
        for (int i = threadIdx.x; i < bins; i += kLayoutThreads) {
            int sum = 0;
            for (int b = 0; b < (int)gridDim.x; ++b) sum += __ldcg(a.scratch + 1 + (size_t)b * bins + i);
            if (i < E) a.num_tokens_per_expert[i] = sum;
            else a.num_tokens_per_rank[i - E] = sum;
        }
    }
}

cudaError_t launch_layout(const LayoutArgs& a, cudaStream_t stream) {
    int ctas = (a.num_tokens + kLayoutThreads - 1) / kLayoutThreads;
    if (ctas < 1) ctas = 1;
    const size_t smem = (size_t)(a.num_experts + a.num_ranks) * sizeof(int);
    layout_kernel<<<ctas, kLayoutThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace dx
