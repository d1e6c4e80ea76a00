// Row gather kernels that move dispatch results into the expert-major, 128-row-aligned layout the grouped
// GEMM wants, and back (weighted) into receive order for combine.
//
//   gather_rows:          dst[m] = scale[m] * src[src_row[m]]            (src_row < 0 -> zero row)
//   gather_reduce_rows:   dst[n] = sum_k w[n,k] * src[pos[n,k]]          (pos < 0 skipped), fp32 accumulate
//
// Both are pure bandwidth kernels: one warp per output row, 16-byte accesses, no atomics. They are each
// other's backward pass, so training needs nothing else.
//
// The reference has no counterpart: its users permute with framework indexing ops between dispatch and
// their expert GEMMs.
#include <cuda_bf16.h>

#include "gemm_api.h"
#include "prims.cuh"

namespace dx {

constexpr int kPermThreads = 256;

// Generic byte rows (any dtype); optional per-row fp32 scale is only legal for bf16 payloads.
__global__ void __launch_bounds__(kPermThreads) gather_rows_kernel(const char* __restrict__ src, char* __restrict__ dst,
                                                                  const int* __restrict__ src_row, const float* __restrict__ scale,
                                                                  int num_dst_rows, int row_bytes) {
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * (kPermThreads / 32) + (threadIdx.x >> 5);
    if (m >= num_dst_rows) return;
    const int s = src_row[m];
    const int n16 = row_bytes / 16;
    int4* d = reinterpret_cast<int4*>(dst + (size_t)m * row_bytes);
    if (s < 0) {
        for (int i = lane; i < n16; i += 32) d[i] = make_int4(0, 0, 0, 0);
        return;
    }
    const int4* p = reinterpret_cast<const int4*>(src + (size_t)s * row_bytes);
    const float sc = scale != nullptr ? scale[m] : 1.f;
    constexpr int U = 4;
    for (int i0 = 0; i0 < n16; i0 += 32 * U) {
        int4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * 32 + lane;
            if (i < n16) v[u] = ld_stream(p + i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * 32 + lane;
            if (i >= n16) continue;
            if (scale != nullptr) {
                uint32_t w[4] = {(uint32_t)v[u].x, (uint32_t)v[u].y, (uint32_t)v[u].z, (uint32_t)v[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = bf16x2_to_f2(w[j]);
                    w[j] = f2_to_bf16x2(f.x * sc, f.y * sc);
                }
                v[u] = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
            }
            d[i] = v[u];
        }
    }
}

__global__ void __launch_bounds__(kPermThreads) gather_reduce_rows_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                                         const int* __restrict__ pos, const float* __restrict__ w,
                                                                         int num_dst_rows, int num_k, int hidden) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (kPermThreads / 32) + (threadIdx.x >> 5);
    if (n >= num_dst_rows) return;
    const int n16 = hidden / 8;
    int my_pos = -1;
    float my_w = 0.f;
    if (lane < num_k) {
        my_pos = pos[(size_t)n * num_k + lane];
        my_w = w != nullptr ? w[(size_t)n * num_k + lane] : 1.f;
    }
    const unsigned valid = __ballot_sync(0xffffffffu, my_pos >= 0);
    int4* d = reinterpret_cast<int4*>(dst) + (size_t)n * n16;
    for (int i = lane; i < n16; i += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        unsigned rest = valid;
        while (rest) {
            const int k = __ffs(rest) - 1;
            rest &= rest - 1;
            const int p = __shfl_sync(0xffffffffu, my_pos, k);
            const float wk = __shfl_sync(0xffffffffu, my_w, k);
            const int4 v = ld_stream(reinterpret_cast<const int4*>(src) + (size_t)p * n16 + i);
            const uint32_t u[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = bf16x2_to_f2(u[j]);
                acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
                acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
            }
        }
        int4 o;
        o.x = (int)f2_to_bf16x2(acc[0], acc[1]);
        o.y = (int)f2_to_bf16x2(acc[2], acc[3]);
        o.z = (int)f2_to_bf16x2(acc[4], acc[5]);
        o.w = (int)f2_to_bf16x2(acc[6], acc[7]);
        d[i] = o;
    }
}

// Expert-major slot assignment: selection (n, k) of local expert e gets row m_offsets[e] + (arrival order among the
// selections of e). Which selection gets which row inside an expert does not matter (rows are independent in the
// GEMM and the inverse map is built in the same pass), so slots are claimed with warp-aggregated atomics.
__global__ void __launch_bounds__(256) build_plan_kernel(const int64_t* __restrict__ topk_idx, const int* __restrict__ m_offsets,
                                                        int* __restrict__ counters, int* __restrict__ pos, int* __restrict__ src_row,
                                                        int* __restrict__ src_k, int num_pairs, int num_topk, int num_local_experts) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int e = -1;
    if (i < num_pairs) {
        const int64_t v = topk_idx[i];
        if (v >= 0 && v < num_local_experts) e = (int)v;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    int p = -1;
    if (e >= 0) {
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if (lane == leader) base = atomicAdd(&counters[e], __popc(peers));
        base = __shfl_sync(peers, base, leader);
        const int slot = base + __popc(peers & ((1u << lane) - 1));
        const int row = m_offsets[e] + slot;
        if (row < m_offsets[e + 1]) {  // cannot overflow when the offsets come from the dispatch counts
            p = row;
            src_row[row] = i / num_topk;
            src_k[row] = i % num_topk;
        }
    }
    if (i < num_pairs) pos[i] = p;
}

cudaError_t launch_build_plan(const int64_t* topk_idx, const int* m_offsets, int* counters, int* pos, int* src_row, int* src_k,
                              int num_rows, int num_topk, int num_local_experts, int m_pad, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(int) * num_local_experts, stream);
    if (e != cudaSuccess) return e;
    if (m_pad > 0) {
        e = cudaMemsetAsync(src_row, 0xFF, sizeof(int) * (size_t)m_pad, stream);  // -1 = padding
        if (e != cudaSuccess) return e;
        e = cudaMemsetAsync(src_k, 0, sizeof(int) * (size_t)m_pad, stream);
        if (e != cudaSuccess) return e;
    }
    const int pairs = num_rows * num_topk;
    if (pairs <= 0) return cudaSuccess;
    build_plan_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(topk_idx, m_offsets, counters, pos, src_row, src_k, pairs, num_topk,
                                                              num_local_experts);
    return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* src, void* dst, const int* src_row, const float* scale, int num_dst_rows, int row_bytes,
                               cudaStream_t stream) {
    if (num_dst_rows <= 0) return cudaSuccess;
    if (row_bytes % 16 != 0) return cudaErrorInvalidValue;
    const int rows_per_cta = kPermThreads / 32;
    gather_rows_kernel<<<(num_dst_rows + rows_per_cta - 1) / rows_per_cta, kPermThreads, 0, stream>>>(
        static_cast<const char*>(src), static_cast<char*>(dst), src_row, scale, num_dst_rows, row_bytes);
    return cudaGetLastError();
}

cudaError_t launch_gather_reduce_rows(const void* src, void* dst, const int* pos, const float* w, int num_dst_rows, int num_k, int hidden,
                                      cudaStream_t stream) {
    if (num_dst_rows <= 0) return cudaSuccess;
    if (hidden % 8 != 0 || num_k > 32 || num_k < 1) return cudaErrorInvalidValue;
    const int rows_per_cta = kPermThreads / 32;
    gather_reduce_rows_kernel<<<(num_dst_rows + rows_per_cta - 1) / rows_per_cta, kPermThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), pos, w, num_dst_rows, num_k, hidden);
    return cudaGetLastError();
}

}  // namespace dx
