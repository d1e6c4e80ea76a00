// Host-visible launch API of the CUDA kernels. No torch headers here: the kernels are plain CUDA and
// the torch binding layer (csrc/host) fills these argument blocks from tensors.
//
// Every kernel that waits on another rank takes an ARRAY of per-rank argument blocks. A real
// multi-process run passes one block (this process' rank). The single-GPU emulation passes one block
// per emulated rank and the kernel is launched cooperatively with gridDim.y = number of ranks, so all
// emulated ranks are co-resident in ONE launch (ranks that wait on each other must never be separate
// launches on one GPU).
//
// Reference counterpart of this file: csrc/kernels/api.cuh:10-348 (namespaces layout / intranode /
// internode_ll) — same responsibilities, different decomposition.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cuda_bf16.h>

#include "types.h"

namespace dx {

// ---- layout -------------------------------------------------------------------------------
struct LayoutArgs {
    const int64_t* topk_idx;      // [T,K], -1 = unselected
    int num_tokens, num_topk, num_experts, num_ranks;
    int* num_tokens_per_rank;     // [R]
    int* num_tokens_per_expert;   // [E]
    bool* is_token_in_rank;       // [T,R]
    int* scratch;                 // >= layout_scratch_ints(E,R,T) ints, first int must be 0 between calls
    // groups that span several NVLink domains: R <= 64 ranks in domains of ranks_per_node; 0 = single domain
    int ranks_per_node;
    int* num_tokens_per_node;     // [R / ranks_per_node] or nullptr
};
size_t layout_scratch_ints(int num_experts, int num_ranks, int num_tokens, int num_nodes = 0);
cudaError_t launch_layout(const LayoutArgs& a, cudaStream_t stream);

// ---- normal mode --------------------------------------------------------------------------
struct NotifyArgs {
    RankCtx ctx;
    const int* num_tokens_per_rank;     // [R]
    const int* num_tokens_per_expert;   // [E]
    const bool* is_token_in_rank;       // [T,R]
    int num_tokens, num_experts, num_channels, expert_alignment;
    int* rank_prefix_matrix;            // [R,R] out
    int* channel_prefix_matrix;         // [R,C] out
    int* recv_channel_prefix_matrix;    // [R,C] out
    int* send_head;                     // [T,R] out: position inside the (me -> r) stream or -1
    volatile int* host_recv_counter;    // mapped host: total rows I will receive
    volatile int* host_expert_counter;  // mapped host [L]: rows per local expert (aligned)
};
cudaError_t launch_notify(const NotifyArgs* a, int num_virtual, cudaStream_t stream);

struct DispatchArgs {
    RankCtx ctx;
    const void* x;                // [T,hidden] bf16, or e4m3 when x_scales != nullptr
    const float* x_scales;        // [T,hidden/128] or nullptr
    int x_elem_bytes;             // 2 (bf16) or 1 (e4m3)
    int quantize;                 // 1: x is bf16 and rows are cast to e4m3 + scales on the fly
    int round_scale;              // power-of-two scales when quantizing
    const int64_t* topk_idx;      // [T,K] or nullptr (cached mode)
    const float* topk_weights;    // [T,K] or nullptr
    int num_topk;
    const int* send_head;         // [T,R]
    const int* rank_prefix_matrix;  // [R,R]
    int num_tokens, hidden, num_experts;
    int num_sms;
    // Where MY received rows go (offsets inside my symmetric buffer); published to all peers.
    uint64_t recv_x_off, recv_scales_off, recv_topk_idx_off, recv_topk_w_off, recv_src_idx_off;
    int num_worst_tokens;         // >0: fill recv_topk_idx rows [num_recv, num_worst_tokens) with -1
};
cudaError_t launch_dispatch(const DispatchArgs* a, int num_virtual, cudaStream_t stream);

struct CombineArgs {
    RankCtx ctx;
    uint64_t x_off;               // my expert outputs [N_recv,hidden] bf16 inside my symmetric buffer
    uint64_t topk_w_off;          // my [N_recv,K] f32 weights inside my symmetric buffer, or ~0
    const int* send_head;         // [T,R] from the dispatch handle
    const int* rank_prefix_matrix;  // [R,R]
    const __nv_bfloat16* bias0;   // [T,hidden] or nullptr
    const __nv_bfloat16* bias1;
    __nv_bfloat16* out;           // [T,hidden]
    float* out_topk_w;            // [T,K] or nullptr
    int num_tokens, hidden, num_topk;
    int num_sms;
};
cudaError_t launch_combine(const CombineArgs* a, int num_virtual, cudaStream_t stream);

struct BarrierArgs {
    RankCtx ctx;
};
cudaError_t launch_barrier(const BarrierArgs* a, int num_virtual, cudaStream_t stream);

// A wait that nothing satisfies, with the caller's (short) limit: proves that a timed-out wait sets
// the status word and returns instead of hanging.
cudaError_t launch_timeout_probe(const RankCtx& ctx, uint64_t* never_set_flag, cudaStream_t stream);

// ---- two-level (NVLink domain x rail) bookkeeping, hier.cu ----------------------------------
struct RoutingSortArgs {
    const bool* member;   // [T, G * ranks_per_group]: token t goes to group g if any of the group's ranks is set
    int num_tokens, num_groups, ranks_per_group;
    int* sorted_ids;      // [sum counts] token ids ordered by (group, token)
    int* counts;          // [G]
    int* prefix;          // [G+1] exclusive prefix of counts
    int* pos;             // [T, G] slot of (t, g) in sorted_ids or -1; may be nullptr
};
cudaError_t launch_routing_sort(const RoutingSortArgs& a, cudaStream_t stream);

struct TopkRemapArgs {
    const int64_t* topk_idx;     // [T, K] global expert ids, -1 = unselected
    const float* topk_weights;   // [T, K] or nullptr
    const int* sorted_ids;       // [S]
    const int* prefix;           // [G+1]
    int num_entries, num_topk, num_groups, experts_per_group;
    uint8_t* packed;             // [S, K*12]: K int64 group-relative ids (or -1), then K f32 weights (or 0)
};
cudaError_t launch_topk_remap_pack(const TopkRemapArgs& a, cudaStream_t stream);

struct RecvSrcMetaArgs {
    const int* recv_prefix;            // [G+1] exclusive prefix of rows received per source group
    const bool* is_row_in_local_rank;  // [n, P] or nullptr
    int num_rows, num_groups, num_local_ranks;
    int* meta;                         // [n, 2] = (source group, bitmask of local ranks)
};
cudaError_t launch_recv_src_meta(const RecvSrcMetaArgs& a, cudaStream_t stream);

struct SegmentedCopyArgs {
    const uint8_t* src;
    uint8_t* dst;
    const int64_t* segments;  // [n, 3] = (src byte offset, dst byte offset, bytes)
    int num_segments;
};
cudaError_t launch_segmented_copy(const SegmentedCopyArgs& a, cudaStream_t stream);

// ---- expert-major dispatch of the fused MoE layer (fused.cu) -----------------------------------
struct EmNotifyArgs {
    RankCtx ctx;
    const int64_t* topk_idx;      // [T,K] global expert ids, -1 = unselected
    int num_tokens, num_topk, num_experts;
    int unit_rows;                // rows per work unit of the dispatch kernel
    int rows_cap;                 // rows every rank's receive buffers hold (the same on all ranks)
    // where MY received rows, their scales, their (source rank, selection) words and my combine stage live (offsets inside
    // my symmetric buffer); published to all peers with the counts
    uint64_t recv_x_off, recv_scales_off, recv_info_off, stage_off;
    // outputs, rank-local device memory
    int* my_counts;               // [E] my selections per expert
    int* sel_list;                // [E, T] selection ids (t*K + k) of every expert in token order
    int* send_base;               // [E] row of my first selection of expert e inside e's rank
    int* unit_start;              // [E+1] exclusive prefix of work units in send order (local expert major, rank minor)
    int* unit_counter;            // [1] next work unit of the dispatch kernel, reset here
    int* m_offsets;               // [L+1] 128-aligned first row of my local experts; [L] = rows in use
    int* m_ends;                  // [L] end of the valid rows of every local expert
    uint64_t* peer_bases;         // [4, R] device pointers of every rank's rows / scales / info / stage
};
cudaError_t launch_em_notify(const EmNotifyArgs* a, int num_virtual, cudaStream_t stream);

struct EmDispatchArgs {
    RankCtx ctx;
    const void* x;                // [T, hidden] bf16 (quantised here), or e4m3 when x_scales is set (copied)
    const float* x_scales;        // [T, hidden/128] f32 scales of pre-quantised rows (powers of two when native_atoms), or nullptr
    int num_tokens, hidden, num_topk, num_experts;
    int unit_rows, round_scale;
    int native_atoms;             // 1: scales are written as the UE8M0 words of [row tile][K block][512] scale atoms
    const int* my_counts;
    const int* sel_list;
    const int* send_base;
    const int* unit_start;
    int* unit_counter;            // [1] next unit to hand out (zeroed by the count exchange)
    const uint64_t* peer_bases;
    int* dst_row;                 // [T*K] or nullptr: row each selection was stored to (entries of unselected slots untouched)
    int num_sms;
    unsigned long long* trace;    // optional [2]: earliest start / latest end of the kernel (global timer, ns)
};
cudaError_t launch_em_dispatch(const EmDispatchArgs* a, int num_virtual, cudaStream_t stream);

// out[t] = sum_k w[t,k] * stage[t*K + k] over the selections with a valid expert id (bf16 rows, fp32 accumulation)
cudaError_t launch_stage_reduce(const void* stage, void* out, const int64_t* topk_idx, const float* w, int num_tokens, int num_topk,
                                int num_experts, int hidden, cudaStream_t stream);

// ---- standalone FP8 cast ------------------------------------------------------------------
struct Fp8CastArgs {
    const __nv_bfloat16* x;   // [M,hidden]
    uint8_t* out;             // [M,hidden] e4m3
    float* scales;            // [M,hidden/128] f32 (when ue8m0 == 0)
    int32_t* scales_ue8m0;    // [M,hidden/512] packed exponents (when ue8m0 == 1)
    int num_rows, hidden;
    int round_scale, ue8m0;
    // optional masking for grouped layouts: row r is cast only if (r % rows_per_group) < group_counts[r / rows_per_group]
    const int* group_counts;
    int rows_per_group;
    const int* num_rows_dev;  // optional device int: only rows below it are cast (a count known on the device only)
    uint8_t* sf_atoms;        // optional: scales go out as UE8M0 scale atoms [ceil(M/128)][hidden/128][512] (power-of-two scales)
};
cudaError_t launch_fp8_cast(const Fp8CastArgs& a, cudaStream_t stream);

// ---- low-latency mode ---------------------------------------------------------------------
// Symmetric low-latency region (same offsets on every rank), two parities.
struct LLRegion {
    uint64_t counts_off[2];       // int [R][E]: counts_off[p] + src*E*4 : how many rows src sends to expert e
    uint64_t recv_x_off[2];       // [L][N][hidden * elem] dispatch payload landing zone (= packed_recv_x)
    uint64_t recv_scales_off[2];  // [L][N][hidden/128] f32
    uint64_t recv_src_info_off[2];// [L][N] int
    uint64_t combine_stage_off[2];// [E][max_tokens][hidden] bf16: rows returned to the home rank
    uint64_t combine_src_off[2];  // [L][N][hidden] bf16: zero-copy combine input buffer
};

struct LLDispatchArgs {
    RankCtx ctx;
    int parity;
    LLRegion region;
    const __nv_bfloat16* x;       // [T,hidden]
    const int64_t* topk_idx;      // [T,K]
    int num_tokens, hidden, num_topk, num_experts, num_max_tokens;
    int use_fp8, round_scale, use_ue8m0;
    int phases;                   // bit0 = send, bit1 = recv
    // outputs (rank-local device memory)
    int* packed_recv_count;       // [L]
    int64_t* layout_range;        // [L,R]
    int* cumulative_stats;        // [L] or nullptr
    int64_t* wait_cost_stats;     // [R] or nullptr
    int* send_row;                // [T,K] or nullptr: row of each selection inside its expert's [N, hidden] block at the expert's rank
                                  // (-1 = not sent); the pull form of combine reads the output row back from there
    int num_sms;
};
cudaError_t launch_ll_dispatch(const LLDispatchArgs* a, int num_virtual, cudaStream_t stream);

struct LLCombineArgs {
    RankCtx ctx;
    int parity;
    LLRegion region;
    const __nv_bfloat16* x;       // [L,N,hidden] expert outputs (rank-local memory or the zero-copy buffer)
    const int64_t* topk_idx;      // [T,K]
    const float* topk_weights;    // [T,K]
    const int* src_info;          // [L,N]
    const int64_t* layout_range;  // [L,R]
    __nv_bfloat16* out;           // [T,hidden] device memory or pinned host memory
    int64_t* wait_cost_stats;     // [R] or nullptr
    int num_tokens, hidden, num_topk, num_experts, num_max_tokens;
    int phases;
    int num_sms;
    // pull form (x lives in this rank's symmetric buffer, every rank's in its own): x_off is posted to the home ranks,
    // which read the rows in place; send_row [T,K] comes from the dispatch of the same handle
    int pull;
    uint64_t x_off;
    const int* send_row;
    int close_barrier;            // pull form: readers report back before the kernel ends (x is a caller-owned tensor)
};
cudaError_t launch_ll_combine(const LLCombineArgs* a, int num_virtual, cudaStream_t stream);

}  // namespace dx
