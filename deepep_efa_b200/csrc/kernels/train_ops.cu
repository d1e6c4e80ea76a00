// Elementwise / layout kernels of the MoE training step that sit between the grouped GEMMs:
//
//   transpose_bf16     batched [B, R, C] -> [B, C, R] through 64x64 shared-memory tiles (16-byte global accesses both ways);
//                      the weight-gradient GEMM reduces over tokens and wants them contiguous, the input-gradient GEMM wants
//                      the weights with their output dimension contiguous
//   swiglu_fwd / bwd   h = silu(gate) * up from h13 = [gate | up], and its gradient, in one pass each (fp32 math, bf16 I/O)
//   rowdot             d_w[n, k] = <a[pos[n, k]], b[n]>  (gradient of the gate weights through the weighted un-permute)
//
// The reference has no counterpart (it ships no model code); these replace chains of framework ops whose copies
// dominated the training step.
#include "gemm_api.h"

#include <cuda_bf16.h>

namespace dx {

namespace {

constexpr int kTile = 64;

__global__ void __launch_bounds__(256) transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int R, int C) {
    // 64x64 tile without padding; the 16-byte chunk `ch` of row r lives at chunk position ch ^ ((r >> 3) & 7). Rows that are a
    // multiple of 8 apart (what the lanes of the store phase read together) then sit in different banks, and the 8 lanes
    // that fill one row in the load phase still cover it exactly once.
    __shared__ __align__(16) __nv_bfloat16 tile[kTile][kTile];
    const size_t plane = (size_t)R * C;
    const __nv_bfloat16* src = in + blockIdx.z * plane;
    __nv_bfloat16* dst = out + blockIdx.z * plane;
    const int r0 = blockIdx.y * kTile, c0 = blockIdx.x * kTile;
    const int tid = threadIdx.x;
    for (int i = tid; i < kTile * 8; i += 256) {
        const int r = i >> 3, ch = i & 7;
        int4 v = make_int4(0, 0, 0, 0);
        if (r0 + r < R && c0 + ch * 8 < C) v = *reinterpret_cast<const int4*>(src + (size_t)(r0 + r) * C + c0 + ch * 8);
        *reinterpret_cast<int4*>(&tile[r][(ch ^ ((r >> 3) & 7)) * 8]) = v;
    }
    __syncthreads();
    // store: output row = input column c; lane (i & 7) = q assembles input rows 8q..8q+7 into one 16-byte chunk, so 8
    // consecutive lanes write one full 128-byte output row segment
    for (int i = tid; i < kTile * 8; i += 256) {
        const int c = i >> 3, q = i & 7;
        if (c0 + c >= C || r0 + q * 8 >= R) continue;
        const int col = (((c >> 3) ^ q) << 3) + (c & 7);  // (r >> 3) & 7 == q for the rows 8q..8q+7
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = tile[q * 8 + j][col];
        *reinterpret_cast<int4*>(dst + (size_t)(c0 + c) * R + r0 + q * 8) = *reinterpret_cast<const int4*>(v);
    }
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ h13, __nv_bfloat16* __restrict__ h, long long rows, int inter) {
    const int chunks = inter / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * chunks; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / chunks;
        const int c = (int)(i % chunks) * 8;
        const int4 g = *reinterpret_cast<const int4*>(h13 + r * 2 * inter + c);
        const int4 u = *reinterpret_cast<const int4*>(h13 + r * 2 * inter + inter + c);
        const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(&g);
        const __nv_bfloat16* up = reinterpret_cast<const __nv_bfloat16*>(&u);
        __align__(16) __nv_bfloat16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(silu_f(__bfloat162float(gp[j])) * __bfloat162float(up[j]));
        *reinterpret_cast<int4*>(h + r * inter + c) = *reinterpret_cast<const int4*>(o);
    }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ h13, const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dh13,
                                  long long rows, int inter) {
    const int chunks = inter / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows * chunks; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / chunks;
        const int c = (int)(i % chunks) * 8;
        const int4 g = *reinterpret_cast<const int4*>(h13 + r * 2 * inter + c);
        const int4 u = *reinterpret_cast<const int4*>(h13 + r * 2 * inter + inter + c);
        const int4 d = *reinterpret_cast<const int4*>(dh + r * inter + c);
        const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(&g);
        const __nv_bfloat16* up = reinterpret_cast<const __nv_bfloat16*>(&u);
        const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(&d);
        __align__(16) __nv_bfloat16 og[8], ou[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float x = __bfloat162float(gp[j]), uu = __bfloat162float(up[j]), dd = __bfloat162float(dp[j]);
            const float sig = 1.f / (1.f + __expf(-x));
            og[j] = __float2bfloat16(dd * uu * sig * (1.f + x * (1.f - sig)));  // d silu(x)/dx = sig * (1 + x * (1 - sig))
            ou[j] = __float2bfloat16(dd * x * sig);
        }
        *reinterpret_cast<int4*>(dh13 + r * 2 * inter + c) = *reinterpret_cast<const int4*>(og);
        *reinterpret_cast<int4*>(dh13 + r * 2 * inter + inter + c) = *reinterpret_cast<const int4*>(ou);
    }
}

// one warp per (n, k)
__global__ void __launch_bounds__(256) rowdot_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, const int* __restrict__ pos,
                                                     float* __restrict__ out, int n_rows, int num_k, int hidden) {
    const int lane = threadIdx.x & 31;
    const long long total = (long long)n_rows * num_k;
    for (long long p = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); p < total; p += (long long)gridDim.x * 8) {
        const int src = pos[p];
        float acc = 0.f;
        if (src >= 0) {
            const int4* ar = reinterpret_cast<const int4*>(a + (size_t)src * hidden);
            const int4* br = reinterpret_cast<const int4*>(b + (size_t)(p / num_k) * hidden);
            const int n16 = hidden / 8;
            constexpr int U = 4;  // four column chunks of both rows in flight per lane
            for (int i0 = 0; i0 < n16; i0 += 32 * U) {
                int4 x[U], y[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    x[u] = i < n16 ? ar[i] : make_int4(0, 0, 0, 0);
                    y[u] = i < n16 ? br[i] : make_int4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x[u]);
                    const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y[u]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 xf = __bfloat1622float2(xp[j]), yf = __bfloat1622float2(yp[j]);
                        acc = fmaf(xf.x, yf.x, fmaf(xf.y, yf.y, acc));
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[p] = acc;
    }
}

}  // namespace

cudaError_t launch_transpose_bf16(const void* in, void* out, int batch, int rows, int cols, cudaStream_t stream) {
    if (batch <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
    if ((rows & 7) != 0 || (cols & 7) != 0 || batch > 65535) return cudaErrorInvalidValue;
    dim3 grid((cols + kTile - 1) / kTile, (rows + kTile - 1) / kTile, batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    transpose_bf16_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), rows, cols);
    return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const void* h13, void* h, long long rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    if ((inter & 7) != 0) return cudaErrorInvalidValue;
    const long long work = rows * (inter / 8);
    const int blocks = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    swiglu_fwd_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h13), static_cast<__nv_bfloat16*>(h), rows, inter);
    return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* h13, const void* dh, void* dh13, long long rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    if ((inter & 7) != 0) return cudaErrorInvalidValue;
    const long long work = rows * (inter / 8);
    const int blocks = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
    swiglu_bwd_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h13), static_cast<const __nv_bfloat16*>(dh),
                                                  static_cast<__nv_bfloat16*>(dh13), rows, inter);
    return cudaGetLastError();
}

cudaError_t launch_rowdot(const void* a, const void* b, const int* pos, float* out, int n_rows, int num_k, int hidden, cudaStream_t stream) {
    const long long total = (long long)n_rows * num_k;
    if (total <= 0) return cudaSuccess;
    if ((hidden & 7) != 0) return cudaErrorInvalidValue;
    const int blocks = (int)((total + 7) / 8 < 148 * 8 ? (total + 7) / 8 : 148 * 8);
    rowdot_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), pos, out, n_rows, num_k, hidden);
    return cudaGetLastError();
}

}  // namespace dx
