// Launch API of the grouped expert GEMM (tcgen05 / TMEM / TMA, sm_100a). No torch headers.
//
//   C[m, n] = sum_k A[m, k] * B[n, k]        (both operands K-major, fp32 accumulation in TMEM)
//
// mode 0, "M-grouped" (expert forward and input gradients): A is [M_total, K]; rows
//   [m_offsets[g], m_offsets[g+1]) belong to expert g and use weight block B[g*N : (g+1)*N, :].
//   Group boundaries must be multiples of 128 (dispatch's expert alignment / the permute pads).
// mode 1, "K-grouped" (weight gradients): A is [N_out, M_total], B is [K_out, M_total]; expert g
//   reduces over columns [m_offsets[g], m_offsets[g+1]) and writes C[g*N_out : (g+1)*N_out, :].
//
// Operand types: BF16 (kind::f16) or FP8 e4m3 with DeepSeek-style scales (one fp32 per 1x128 of A and
// per 128x128 of B): every 128-deep K block is accumulated in its own TMEM window and promoted into
// fp32 registers with the product of the two scales.
// swiglu = 1: B holds [gate; up] stacked per expert ([G, 2*I, K]); a tile computes matching gate and up
//   columns and writes silu(gate) * up, so C is [M_total, I].
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dx {

struct GroupedGemmArgs {
    const void* a;            // operand A (see mode)
    const void* b;            // operand B
    void* c;                  // bf16 output
    const float* a_scales;    // fp8 only: [M_total, K/128]
    const float* b_scales;    // fp8 only: [G, N/128, K/128]
    // fp8 with native block scaling (power-of-two scales; mode 0, group starts on multiples of 128 rows): UE8M0 scale atoms,
    // 512 bytes per (128 rows, 128 K): [ceil(M/128)][K/128][512] and [G][N/128 tiles (swiglu: N/2/64 tiles)][K/128][512];
    // when sfa_atoms is set the fp32 scale pointers are ignored
    const uint8_t* sfa_atoms;
    const uint8_t* sfb_atoms;
    int mx_wide;              // swiglu only: 1 = 256-column tiles (one accumulator window; large groups), 0 = 128-column tiles
    const int* m_offsets;     // [G+1] device memory
    const int* m_ends;        // optional [G]: group g covers rows [m_offsets[g], m_ends[g]) instead of up to m_offsets[g+1]
                              // (mode 0 only; the low-latency layout has fixed group starts and a count per expert)
    int num_groups;
    int mode;                 // 0 = M-grouped, 1 = K-grouped
    int fp8;                  // 0 = bf16 operands, 1 = e4m3 operands (mode 0 only)
    int swiglu;               // mode 0 only
    int m_total;              // rows of A (mode 0) / reduction length (mode 1)
    int n;                    // mode 0: rows of B per expert (2*I when swiglu); mode 1: N_out (rows of A)
    int k;                    // mode 0: reduction length; mode 1: K_out (rows of B)
    int num_sms;              // persistent grid size
    int tile_order;           // mode 0: 0 = weight tile shared by consecutive CTAs, 1 = activation tile shared
    int cta_pairs;            // 1 = two CTAs of a cluster share one 256-row MMA (cta_group::2), each staging half of the B tile
    int* error_flag;          // device int, set non-zero when a bounded pipeline wait ran out
    long long timeout_cycles;
    // Arrival gating (mode 0): the rows of group g are written by other GPUs while this kernel runs. Before the first tile
    // of a group is loaded, the loader waits (bounded) until ready[g] >= expected[g]; `ready` is advanced with system-scope
    // release reductions by the senders, `expected` is rank-local. Both null = no gating.
    const unsigned long long* ready;
    const unsigned long long* expected;
    // Scatter epilogue (mode 0, no swiglu): output row m is not stored to c[m] but to row (row_info[m] & 0xffffff) of the
    // [rows, n] bf16 matrix at scatter_bases[row_info[m] >> 24] (a peer's symmetric memory or this GPU's); rows whose word
    // is negative are dropped. Null = ordinary output.
    const int* row_info;
    const unsigned long long* scatter_bases;
    unsigned long long* trace;  // optional [4]: earliest first-tile load / latest epilogue end (global timer, ns) / first wait that
                                // gave up (role << 56 | tile << 24 | k block << 8 | slot; 0 = none) / what the loader was doing
                                // then (state << 32 | tile; state 1 = arrival gate, 2 = waiting for a free stage, 3 = loads issued)
    // MN-major operands (bf16, no swiglu): the operand is read from a tensor whose contiguous dimension is the operand's row
    // index instead of K, so gradients need no transposed copies. mode 0: b_mn = 1, B given as [G, K, N] (input gradients:
    // the forward weight as it is). mode 1: a_mn = b_mn = 1, A given as [M_total, N_out], B as [M_total, K_out] (weight
    // gradients: output gradient and activation as they are).
    int a_mn, b_mn;
    // Quantised output (natively block-scaled kernel with 256-column SwiGLU tiles only): instead of bf16 rows in `c`, write
    // e4m3 rows [M_total, N/2] to c_fp8 and their power-of-two scales as UE8M0 scale atoms [ceil(M/128)][N/2/128][512] to
    // c_atoms: the activation operand of the next natively block-scaled GEMM, without a cast pass in between.
    uint8_t* c_fp8;
    uint8_t* c_atoms;
};

// Returns cudaErrorInvalidValue for unsupported shapes (divisibility rules are in grouped_gemm.cu).
cudaError_t launch_grouped_gemm(const GroupedGemmArgs& args, cudaStream_t stream);

// Expert-major plan from local expert ids [N, K] (-1 = unselected) and 128-aligned group offsets [L+1]:
// pos [N*K], src_row [m_pad] (-1 = padding), src_k [m_pad]; counters is an int[L] scratch.
cudaError_t launch_build_plan(const int64_t* topk_idx, const int* m_offsets, int* counters, int* pos, int* src_row, int* src_k,
                              int num_rows, int num_topk, int num_local_experts, int m_pad, cudaStream_t stream);

// Row gathers between receive order and the expert-major, 128-row-aligned layout (permute.cu).
//   dst[m] = scale[m] * src[src_row[m]]   (src_row[m] < 0 -> zero row; scale may be null; bf16 rows when scaled)
cudaError_t launch_gather_rows(const void* src, void* dst, const int* src_row, const float* scale, int num_dst_rows, int row_bytes,
                               cudaStream_t stream);
//   dst[n] = sum_k w[n,k] * src[pos[n,k]]  (bf16 rows, fp32 accumulate; pos < 0 skipped; w may be null = 1)
cudaError_t launch_gather_reduce_rows(const void* src, void* dst, const int* pos, const float* w, int num_dst_rows, int num_k, int hidden,
                                      cudaStream_t stream);

// Training-step helpers (train_ops.cu). All tensors bf16 unless noted.
//   out[b, c, r] = in[b, r, c]                     rows and cols multiples of 8
cudaError_t launch_transpose_bf16(const void* in, void* out, int batch, int rows, int cols, cudaStream_t stream);
//   h[m, i] = silu(h13[m, i]) * h13[m, inter + i]
cudaError_t launch_swiglu_fwd(const void* h13, void* h, long long rows, int inter, cudaStream_t stream);
//   dh13 = d/dh13 of the above given dh
cudaError_t launch_swiglu_bwd(const void* h13, const void* dh, void* dh13, long long rows, int inter, cudaStream_t stream);
//   out[n, k] = <a[pos[n, k]], b[n]>  (f32 out, 0 where pos < 0)
cudaError_t launch_rowdot(const void* a, const void* b, const int* pos, float* out, int n_rows, int num_k, int hidden, cudaStream_t stream);

// Scale atoms of the natively block-scaled FP8 GEMM (sf_atoms.cu); scales must be powers of two.
cudaError_t launch_build_sfa_atoms(const float* scales, uint8_t* atoms, int rows, int num_kb, cudaStream_t stream);
cudaError_t launch_build_sfb_atoms(const float* scales, uint8_t* atoms, int groups, int n, int num_kb, int swiglu, int wide,
                                   cudaStream_t stream);

}  // namespace dx
