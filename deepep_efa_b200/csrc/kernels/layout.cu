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

// bins per CTA: experts, ranks, and one per NVLink domain when those are counted too
size_t layout_scratch_ints(int num_experts, int num_ranks, int num_tokens, int num_nodes) {
    const size_t ctas = (num_tokens + kLayoutThreads - 1) / kLayoutThreads;
    return 1 + (ctas > 0 ? ctas : 1) * (size_t)(num_experts + num_ranks + num_nodes);
}

__global__ void __launch_bounds__(kLayoutThreads) layout_kernel(const LayoutArgs a) {
    extern __shared__ int s_hist[];  // [E] experts, [R] ranks, [R / ranks_per_node] NVLink domains
    const int E = a.num_experts, R = a.num_ranks, K = a.num_topk;
    const int L = E / R;
    const int P = a.ranks_per_node > 0 ? a.ranks_per_node : R;
    const int nodes = a.num_tokens_per_node != nullptr ? R / P : 0;
    const int bins = E + R + nodes;
    for (int i = threadIdx.x; i < bins; i += kLayoutThreads) s_hist[i] = 0;
    __syncthreads();

    const int t = blockIdx.x * kLayoutThreads + threadIdx.x;
    uint64_t mask = 0;
    if (t < a.num_tokens) {
        const int64_t* row = a.topk_idx + (size_t)t * K;
        for (int k = 0; k < K; ++k) {
            const int64_t e = row[k];
            if (e >= 0 && e < E) {
                atomicAdd(&s_hist[(int)e], 1);
                mask |= 1ull << ((int)e / L);
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
    for (int n = 0; n < nodes; ++n) {
        const uint64_t node_bits = (P >= 64 ? ~0ull : ((1ull << P) - 1ull)) << (n * P);
        const unsigned b = __ballot_sync(0xffffffffu, (mask & node_bits) != 0);
        if ((threadIdx.x & 31) == 0 && b) atomicAdd(&s_hist[E + R + n], __popc(b));
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
            else if (i < E + R) a.num_tokens_per_rank[i - E] = sum;
            else a.num_tokens_per_node[i - E - R] = sum;
        }
    }
}

cudaError_t launch_layout(const LayoutArgs& a, cudaStream_t stream) {
    int ctas = (a.num_tokens + kLayoutThreads - 1) / kLayoutThreads;
    if (ctas < 1) ctas = 1;
    if (a.num_ranks > 64) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(a.num_experts + 2 * a.num_ranks) * sizeof(int);  // upper bound of the bins
    layout_kernel<<<ctas, kLayoutThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace dx
