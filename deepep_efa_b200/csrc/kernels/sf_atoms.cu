// Scale-factor atoms for the natively block-scaled FP8 GEMM (tcgen05.mma kind::mxf8f6f4.block_scale).
//
// The tensor core reads one UE8M0 byte (a power-of-two exponent) per row and per 32 K-elements from TMEM. A 128-row x 128-K
// scale tile travels as a 512-byte atom: the byte of row (m0 + 32*m1), K sub-block kb sits at m0*16 + m1*4 + kb, which is
// what tcgen05.cp.32x128b.warpx4 spreads over four TMEM columns. The library's scales have one value per 128 K-elements
// (1x128 on activations, 128x128 on weights), so the four bytes of a word are equal.
//
// These kernels turn fp32 power-of-two scales into atoms:
//   A: scales [M, K/128]          -> [ceil(M/128)][K/128][512]
//   B: scales [G, N/128, K/128]   -> plain: [G][N/128][K/128][512], tiles of 128 B rows;
//                                    SwiGLU, 256-column tiles (wide): [G][N/256][K/128][2][512], a tile is 128 gate rows followed
//                                    by the 128 matching up rows: first atom = the gate rows' scale block, second = the up rows'
//                                    SwiGLU, 128-column tiles: [G][N/128][K/128][512], 64 gate + 64 up rows share one atom
// The reference has no counterpart (no GEMM).
#include "gemm_api.h"

namespace dx {

namespace {

__device__ __forceinline__ uint32_t ue8m0_word(float scale) {
    const uint32_t e = (__float_as_uint(scale) >> 23) & 0xffu;  // biased exponent of a power of two
    return e * 0x01010101u;
}

__global__ void sfa_atoms_kernel(const float* __restrict__ scales, uint8_t* __restrict__ atoms, int rows, int num_kb, long long total) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m0 = (int)(i & 31);
        const long long tk = i >> 5;           // tile * num_kb + kb
        const int kb = (int)(tk % num_kb);
        const long long tile = tk / num_kb;
        uint32_t w[4];
#pragma unroll
        for (int m1 = 0; m1 < 4; ++m1) {
            const long long row = tile * 128 + m0 + 32 * m1;
            w[m1] = row < rows ? ue8m0_word(scales[row * num_kb + kb]) : 127u * 0x01010101u;  // 2^0 for padding rows
        }
        *reinterpret_cast<uint4*>(atoms + tk * 512 + m0 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

__global__ void sfb_atoms_kernel(const float* __restrict__ scales, uint8_t* __restrict__ atoms, int n, int num_kb, int tiles, int swiglu,
                                 int wide, long long total) {
    const int nb = n / 128;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m0 = (int)(i & 31);
        const long long tk = i >> 5;           // (g * tiles + t) * num_kb + kb
        const int kb = (int)(tk % num_kb);
        const long long gt = tk / num_kb;
        const int t = (int)(gt % tiles);
        const long long g = gt / tiles;
        if (swiglu && wide == 0) {
            // 128-column tiles: 64 gate rows then the 64 matching up rows share one atom (m1 = 0,1 gate; 2,3 up)
            const int gate_block = (t * 64) / 128, up_block = (n / 2 + t * 64) / 128;
            const uint32_t wg = ue8m0_word(scales[(g * nb + gate_block) * num_kb + kb]);
            const uint32_t wu = ue8m0_word(scales[(g * nb + up_block) * num_kb + kb]);
            *reinterpret_cast<uint4*>(atoms + tk * 512 + m0 * 16) = make_uint4(wg, wg, wu, wu);
        } else if (swiglu) {
            const uint32_t wg = ue8m0_word(scales[(g * nb + t) * num_kb + kb]);
            const uint32_t wu = ue8m0_word(scales[(g * nb + nb / 2 + t) * num_kb + kb]);
            *reinterpret_cast<uint4*>(atoms + tk * 1024 + m0 * 16) = make_uint4(wg, wg, wg, wg);
            *reinterpret_cast<uint4*>(atoms + tk * 1024 + 512 + m0 * 16) = make_uint4(wu, wu, wu, wu);
        } else if (wide) {
            // 256-column tiles without SwiGLU: the atoms of the two neighbouring 128-row blocks side by side
            const uint32_t w0 = ue8m0_word(scales[(g * nb + 2 * t) * num_kb + kb]);
            const uint32_t w1 = ue8m0_word(scales[(g * nb + 2 * t + 1) * num_kb + kb]);
            *reinterpret_cast<uint4*>(atoms + tk * 1024 + m0 * 16) = make_uint4(w0, w0, w0, w0);
            *reinterpret_cast<uint4*>(atoms + tk * 1024 + 512 + m0 * 16) = make_uint4(w1, w1, w1, w1);
        } else {
            const uint32_t wv = ue8m0_word(scales[(g * nb + t) * num_kb + kb]);
            *reinterpret_cast<uint4*>(atoms + tk * 512 + m0 * 16) = make_uint4(wv, wv, wv, wv);
        }
    }
}

}  // namespace

cudaError_t launch_build_sfa_atoms(const float* scales, uint8_t* atoms, int rows, int num_kb, cudaStream_t stream) {
    const long long tiles = (rows + 127) / 128;
    const long long total = tiles * num_kb * 32;
    if (total <= 0) return cudaSuccess;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    sfa_atoms_kernel<<<blocks, 256, 0, stream>>>(scales, atoms, rows, num_kb, total);
    return cudaGetLastError();
}

cudaError_t launch_build_sfb_atoms(const float* scales, uint8_t* atoms, int groups, int n, int num_kb, int swiglu, int wide,
                                   cudaStream_t stream) {
    if (n % 128 != 0 || (swiglu && (n / 2) % 128 != 0) || (!swiglu && wide && n % 256 != 0)) return cudaErrorInvalidValue;
    const int tiles = swiglu ? (wide ? (n / 2) / 128 : (n / 2) / 64) : (wide ? n / 256 : n / 128);
    const long long total = (long long)groups * tiles * num_kb * 32;
    if (total <= 0) return cudaSuccess;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    sfb_atoms_kernel<<<blocks, 256, 0, stream>>>(scales, atoms, n, num_kb, tiles, swiglu, wide, total);
    return cudaGetLastError();
}

}  // namespace dx
