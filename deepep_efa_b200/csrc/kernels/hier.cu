// Bookkeeping kernels of the two-level (NVLink domain x rail) expert-parallel path.
//
// When a group spans several NVLink domains, a token crosses the inter-domain network once per destination
// DOMAIN (to the rank with the sender's local index there) and is fanned out inside that domain by the NVLink
// dispatch kernel. These kernels build the send plan of the first hop and the metadata of the second one:
//
//   routing_sort      stable counting sort of (token, destination group) pairs by group      -> sorted ids, counts,
//                     exclusive prefix, and the inverse map pos[t, g]
//   topk_remap_pack   per send entry: expert ids relative to the destination group (or -1) and weights (or 0),
//                     packed as one row [K x int64 | K x f32] so that one collective carries both
//   recv_src_meta     per received row: (source group, bitmask of the local ranks it is forwarded to)
//   segmented_copy    byte-granular copy of a list of (src offset, dst offset, bytes) segments
//
// Reference counterparts (csrc/kernels/efa_kernels.cu): moe_routing_sort_kernel + prefix_sum_kernel +
// scatter_token_ids_kernel (:220-318, three launches, the last one single-threaded per rank, ending in a host
// sync), topk_remap_kernel (:339-387), build_recv_src_meta_kernel (:448-482), efa_permute_kernel (:405-435).
// Here the sort is one launch without global atomics or host round trip, and every CTA derives its own base offset.
#include "api.h"
#include "prims.cuh"

namespace dx {

constexpr int kSortThreads = 1024;

__device__ __forceinline__ bool in_group(const bool* member, int t, int g, int ranks_total, int ranks_per_group) {
    const bool* row = member + (size_t)t * ranks_total + (size_t)g * ranks_per_group;
    bool any = false;
    for (int j = 0; j < ranks_per_group; ++j) any |= row[j];
    return any;
}

// Grid = (token chunks of 1024, groups). CTA (b, g) places the members of group g among tokens [1024 b, 1024 b + 1024).
// Its base offset = all pairs of earlier groups + the group's members among earlier tokens, which it counts itself from
// the membership matrix (L2-resident re-reads instead of a second launch or inter-CTA waiting).
__global__ void __launch_bounds__(kSortThreads) routing_sort_kernel(const RoutingSortArgs a) {
    __shared__ int s_warp[32];
    __shared__ int s_base, s_group_total;
    const int g = blockIdx.y, G = a.num_groups, T = a.num_tokens;
    const int t_begin = blockIdx.x * kSortThreads;
    const int ranks_total = G * a.ranks_per_group;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    int before = 0, total = 0;
    for (int t = threadIdx.x; t < T; t += kSortThreads) {
        for (int c = 0; c < g; ++c) before += in_group(a.member, t, c, ranks_total, a.ranks_per_group) ? 1 : 0;
        const int mine = in_group(a.member, t, g, ranks_total, a.ranks_per_group) ? 1 : 0;
        total += mine;
        if (t < t_begin) before += mine;
    }
    before = warp_sum(before);
    total = warp_sum(total);
    if (threadIdx.x == 0) {
        s_base = 0;
        s_group_total = 0;
    }
    __syncthreads();
    if (lane == 0) {
        atomicAdd(&s_base, before);
        atomicAdd(&s_group_total, total);
    }
    __syncthreads();
    const int base = s_base;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        a.counts[g] = s_group_total;
        a.prefix[g] = base;
        if (g == G - 1) a.prefix[G] = base + s_group_total;
    }

    const int t = t_begin + threadIdx.x;
    const bool flag = t < T && in_group(a.member, t, g, ranks_total, a.ranks_per_group);
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int warp_off = 0;
    for (int w = 0; w < warp; ++w) warp_off += s_warp[w];
    if (t < T) {
        const int slot = base + warp_off + __popc(ballot & ((1u << lane) - 1u));
        if (flag) a.sorted_ids[slot] = t;
        if (a.pos != nullptr) a.pos[(size_t)t * G + g] = flag ? slot : -1;
    }
}

cudaError_t launch_routing_sort(const RoutingSortArgs& a, cudaStream_t stream) {
    if (a.num_groups < 1 || a.ranks_per_group < 1) return cudaErrorInvalidValue;
    const int chunks = a.num_tokens > 0 ? (a.num_tokens + kSortThreads - 1) / kSortThreads : 1;
    routing_sort_kernel<<<dim3(chunks, a.num_groups), kSortThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

// group of send entry s: the last g with prefix[g] <= s (prefix has G+1 entries, G <= 64: a linear scan)
__device__ __forceinline__ int group_of_entry(const int* prefix, int G, int s) {
    int g = 0;
    while (g + 1 < G && __ldg(prefix + g + 1) <= s) ++g;
    return g;
}

__global__ void topk_remap_pack_kernel(const TopkRemapArgs a) {
    const int K = a.num_topk;
    const size_t row_bytes = (size_t)K * 12;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)a.num_entries * K; i += (long long)gridDim.x * blockDim.x) {
        const int s = (int)(i / K), k = (int)(i % K);
        const int t = a.sorted_ids[s];
        const int g = group_of_entry(a.prefix, a.num_groups, s);
        const int64_t lo = (int64_t)g * a.experts_per_group;
        const int64_t e = a.topk_idx[(size_t)t * K + k];
        const bool mine = e >= lo && e < lo + a.experts_per_group;
        uint8_t* row = a.packed + (size_t)s * row_bytes;
        reinterpret_cast<int64_t*>(row)[k] = mine ? e - lo : -1;
        reinterpret_cast<float*>(row + (size_t)K * 8)[k] = (mine && a.topk_weights != nullptr) ? a.topk_weights[(size_t)t * K + k] : 0.f;
    }
}

cudaError_t launch_topk_remap_pack(const TopkRemapArgs& a, cudaStream_t stream) {
    const long long n = (long long)a.num_entries * a.num_topk;
    if (n == 0) return cudaSuccess;
    const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
    topk_remap_pack_kernel<<<blocks, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

__global__ void recv_src_meta_kernel(const RecvSrcMetaArgs a) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.num_rows; i += gridDim.x * blockDim.x) {
        const int g = group_of_entry(a.recv_prefix, a.num_groups, i);
        int bits = 0;
        if (a.is_row_in_local_rank != nullptr)
            for (int j = 0; j < a.num_local_ranks; ++j) bits |= (a.is_row_in_local_rank[(size_t)i * a.num_local_ranks + j] ? 1 : 0) << j;
        a.meta[2 * (size_t)i] = g;
        a.meta[2 * (size_t)i + 1] = bits;
    }
}

cudaError_t launch_recv_src_meta(const RecvSrcMetaArgs& a, cudaStream_t stream) {
    if (a.num_rows == 0) return cudaSuccess;
    const int blocks = (a.num_rows + 255) / 256 < 1024 ? (a.num_rows + 255) / 256 : 1024;
    recv_src_meta_kernel<<<blocks, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

// Segments are cut into 32 KiB chunks and the chunks of all segments are dealt round-robin to the CTAs, so that a few
// large segments (one per node in the two-level path) use the whole grid as well as many small ones do.
constexpr int64_t kSegChunk = 32 << 10;

__global__ void __launch_bounds__(256) segmented_copy_kernel(const SegmentedCopyArgs a) {
    const int64_t G = gridDim.x;
    int64_t base = 0;  // chunks of the segments before s
    for (int s = 0; s < a.num_segments; ++s) {
        const int64_t so = a.segments[3 * (size_t)s], d_o = a.segments[3 * (size_t)s + 1], n = a.segments[3 * (size_t)s + 2];
        const int64_t chunks = (n + kSegChunk - 1) / kSegChunk;
        const uint8_t* src = a.src + so;
        uint8_t* dst = a.dst + d_o;
        const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
        for (int64_t c = ((int64_t)blockIdx.x - base % G + G) % G; c < chunks; c += G) {
            const int64_t lo = c * kSegChunk, len = n - lo < kSegChunk ? n - lo : kSegChunk;
            if (vec) {
                const int4* s4 = reinterpret_cast<const int4*>(src + lo);
                int4* d4 = reinterpret_cast<int4*>(dst + lo);
                const int64_t n16 = len / 16;
                int64_t i = threadIdx.x;
                for (; i + 3 * 256 < n16; i += 4 * 256) {
                    const int4 v0 = ld_stream(s4 + i), v1 = ld_stream(s4 + i + 256), v2 = ld_stream(s4 + i + 512), v3 = ld_stream(s4 + i + 768);
                    d4[i] = v0, d4[i + 256] = v1, d4[i + 512] = v2, d4[i + 768] = v3;
                }
                for (; i < n16; i += 256) d4[i] = ld_stream(s4 + i);
                for (int64_t j = n16 * 16 + threadIdx.x; j < len; j += 256) dst[lo + j] = src[lo + j];
            } else {
                for (int64_t j = threadIdx.x; j < len; j += 256) dst[lo + j] = src[lo + j];
            }
        }
        base += chunks;
    }
}

cudaError_t launch_segmented_copy(const SegmentedCopyArgs& a, cudaStream_t stream) {
    if (a.num_segments == 0) return cudaSuccess;
    segmented_copy_kernel<<<1184, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace dx
