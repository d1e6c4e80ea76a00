// Standalone per-token BF16 -> FP8 e4m3 cast with one scale per 128 channels.
//
// The dispatch kernels quantise on the fly; this kernel exists for callers that want the cast alone
// (tests, the FP8 GEMM's activation operand) and is the GPU twin of the pure-torch oracle.
// One warp per row; a lane owns 16 consecutive channels, 8 lanes share a scale group.
// Scales come out as fp32 [M, hidden/128], or as UE8M0 exponent bytes packed four to an int32
// [M, hidden/512] (power-of-two scales only).
//
// Reference counterpart: per_token_cast_to_fp8_kernel, csrc/kernels/efa_kernels.cu:104-187 (grid
// (hidden/128, M) x 128 threads, UE8M0 packing through atomicOr).
#include "api.h"
#include "prims.cuh"

namespace dx {

constexpr int kCastThreads = 256;

__global__ void __launch_bounds__(kCastThreads) fp8_cast_kernel(const Fp8CastArgs a) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (kCastThreads / 32) + (threadIdx.x >> 5);
    if (row >= a.num_rows) return;
    if (a.group_counts != nullptr && (row % a.rows_per_group) >= a.group_counts[row / a.rows_per_group]) return;  // padding row
    if (a.num_rows_dev != nullptr && row >= *a.num_rows_dev) return;
    const int H = a.hidden;
    const char* src = reinterpret_cast<const char*>(a.x) + (size_t)row * H * 2;
    uint8_t* dst = a.out + (size_t)row * H;
    const bool pow2 = a.round_scale != 0 || a.ue8m0 != 0 || a.sf_atoms != nullptr;
    for (int c0 = 0; c0 < H; c0 += 512) {
        const int ch = c0 + lane * 16;
        const bool act = ch < H;
        int4 r0 = make_int4(0, 0, 0, 0), r1 = r0;
        if (act) {
            r0 = ld_cached(reinterpret_cast<const int4*>(src + (size_t)ch * 2));
            r1 = ld_cached(reinterpret_cast<const int4*>(src + (size_t)ch * 2 + 16));
        }
        const uint32_t w[8] = {(uint32_t)r0.x, (uint32_t)r0.y, (uint32_t)r0.z, (uint32_t)r0.w,
                               (uint32_t)r1.x, (uint32_t)r1.y, (uint32_t)r1.z, (uint32_t)r1.w};
        float f[16];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 p = bf16x2_to_f2(w[j]);
            f[2 * j] = p.x;
            f[2 * j + 1] = p.y;
            amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        float scale, inv;
        fp8_scale_from_amax(amax, pow2, scale, inv);
        int4 q;
        q.x = (int)pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
        q.y = (int)pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
        q.z = (int)pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
        q.w = (int)pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
        if (act) *reinterpret_cast<int4*>(dst + ch) = q;
        if (a.sf_atoms != nullptr) {
            if (act && (lane & 7) == 0) {
                const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
                *reinterpret_cast<uint32_t*>(a.sf_atoms + ((size_t)(row >> 7) * (H / 128) + (ch >> 7)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4) =
                    ex * 0x01010101u;
            }
        } else if (a.ue8m0) {
            // lanes 0,8,16,24 hold the four group scales of this 512-channel step
            const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
            const uint32_t e0 = __shfl_sync(0xffffffffu, ex, 0), e1 = __shfl_sync(0xffffffffu, ex, 8);
            const uint32_t e2 = __shfl_sync(0xffffffffu, ex, 16), e3 = __shfl_sync(0xffffffffu, ex, 24);
            if (lane == 0 && c0 + 512 <= H) a.scales_ue8m0[(size_t)row * (H / 512) + c0 / 512] = (int32_t)(e0 | (e1 << 8) | (e2 << 16) | (e3 << 24));
        } else if (act && (lane & 7) == 0) {
            a.scales[(size_t)row * (H / 128) + (ch >> 7)] = scale;
        }
    }
}

cudaError_t launch_fp8_cast(const Fp8CastArgs& a, cudaStream_t stream) {
    if (a.num_rows == 0) return cudaSuccess;
    const int rows_per_cta = kCastThreads / 32;
    fp8_cast_kernel<<<(a.num_rows + rows_per_cta - 1) / rows_per_cta, kCastThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace dx
