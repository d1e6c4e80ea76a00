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
    unsigned valid = __ballot_sync(0xffffffffu, my_pos >= 0);
    int4* d = reinterpret_cast<int4*>(dst) + (size_t)n * n16;
    // Selections compacted onto the low lanes; a row at an expert rank typically has one or two valid selections, so the
    // memory-level parallelism comes from four column chunks per lane being in flight at once.
    const int nv = __popc(valid);
    const int from = lane < nv ? __fns(valid, 0, lane + 1) : 0;
    const int pos_c = __shfl_sync(0xffffffffu, my_pos, from);
    const float w_c = __shfl_sync(0xffffffffu, my_w, from);
    constexpr int U = 4;
    for (int i0 = 0; i0 < n16; i0 += 32 * U) {
        float acc[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
        for (int j = 0; j < nv; ++j) {
            const int pj = __shfl_sync(0xffffffffu, pos_c, j);
            const float wj = __shfl_sync(0xffffffffu, w_c, j);
            const int4* row = reinterpret_cast<const int4*>(src) + (size_t)pj * n16;
            int4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32 + lane;
                v[u] = i < n16 ? ld_stream(row + i) : make_int4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t w4[4] = {(uint32_t)v[u].x, (uint32_t)v[u].y, (uint32_t)v[u].z, (uint32_t)v[u].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = bf16x2_to_f2(w4[q]);
                    acc[u][2 * q] = fmaf(wj, f.x, acc[u][2 * q]);
                    acc[u][2 * q + 1] = fmaf(wj, f.y, acc[u][2 * q + 1]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * 32 + lane;
            if (i >= n16) continue;
            int4 o;
            o.x = (int)f2_to_bf16x2(acc[u][0], acc[u][1]);
            o.y = (int)f2_to_bf16x2(acc[u][2], acc[u][3]);
            o.z = (int)f2_to_bf16x2(acc[u][4], acc[u][5]);
            o.w = (int)f2_to_bf16x2(acc[u][6], acc[u][7]);
            d[i] = o;
        }
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
