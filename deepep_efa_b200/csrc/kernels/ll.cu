// Low-latency dispatch / combine for ~128 tokens per rank over one NVSwitch domain.
//
// dispatch (one launch):
//   * every rank all-gathers its per-expert selection counts (E ints per peer, one release flag),
//   * one CTA per token quantises the row in registers (BF16 -> e4m3, one scale per 128 channels) and
//     stores it K times, straight into the FINAL position of the peers' packed_recv_x: row
//     `sum_{src<me} count[src][e] + slot` of expert e, which every sender can compute from the
//     all-gathered counts. There is no send buffer, no receive-side unpack pass and no memset of
//     the [L, N, hidden] output,
//   * arrival is counted per source rank with monotonic release reductions; the last CTA derives
//     packed_recv_count / layout_range from the counts and waits for the rows.
// combine (one launch): expert ranks push their BF16 rows into the home rank's [E][max_tokens] stage
// (address = (expert, token), so no metadata travels), the home rank waits per source, then one CTA
// per token does sum_k w[t,k] * row in fp32 and writes BF16 once — deterministic order, no atomics.
//
// `phases` splits either kernel into its send (bit 0) and receive (bit 1) half for the
// return_recv_hook contract. Sequence numbers and expected-arrival totals live on the device, so a
// launch carries no per-call value besides the buffer parity.
//
// Reference counterparts: LL route/count/pack kernels + NCCL all-to-all + recv count/build/scatter
// (csrc/kernels/efa_kernels.cu:512-1389, deep_ep/buffer.py:2265-2303), weighted reduce with fp32
// atomics + cast pass (efa_kernels.cu:1413-1486), and the cooperative send/recv kernels
// (csrc/kernels/coop_dispatch_send.cuh, coop_dispatch_recv.cuh, coop_combine_send.cuh,
// coop_combine_recv.cuh).
#include "api.h"
#include "prims.cuh"
#include "launch.cuh"

namespace dx {

constexpr int kLLThreads = 512;
constexpr int kLLWarps = kLLThreads / 32;
constexpr int kTicketLLDispatch = 3;
constexpr int kTicketLLCombine = 4;
// rank-local u64 words after the family sequence numbers (RankCtx::seq + kNumFamilies):
// expected cumulative arrivals [2 kinds][2 parities][kMaxRanks]
__device__ __forceinline__ uint64_t* expected_word(const RankCtx& c, int kind, int parity, int src) {
    return c.seq + kNumFamilies + (kind * 2 + parity) * kMaxRanks + src;
}

// =============================================================================================
// dispatch
// =============================================================================================
template <int V>
__global__ void __launch_bounds__(kLLThreads, 1) ll_dispatch_kernel(const __grid_constant__ ArgPack<LLDispatchArgs, V> pack) {
    const LLDispatchArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk, E = a.num_experts;
    const int L = E / R, H = a.hidden, P = a.parity;
    const int N = R * a.num_max_tokens;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t seq = next_seq(c, kFamLLDispatch);
    const bool do_send = a.phases & 1, do_recv = a.phases & 2;
    const int num_token_ctas = gridDim.x - 1;
    const bool is_tail_cta = blockIdx.x == gridDim.x - 1;
    ControlBlock* my = c.my_ctrl();
    const int* my_counts = c.at<const int>(me, a.region.counts_off[P]);  // [R][E], written by peers

    extern __shared__ int s_mem[];
    int* s_idx = s_mem;              // [T*K] expert id of every selection of this rank
    int* s_hist = s_mem + T * K;     // [E] (tail CTA only)
    __shared__ int s_ok;
    __shared__ int s_row[kMaxTopk];      // destination row inside the expert, -1 = skip
    __shared__ int s_dst_rank[kMaxTopk];
    __shared__ int s_dst_le[kMaxTopk];
    __shared__ int s_sent[kMaxRanks];

    if (tid == 0) s_ok = 1;
    if (tid < kMaxRanks) s_sent[tid] = 0;
    for (int i = tid; i < T * K; i += kLLThreads) {
        const int64_t e = a.topk_idx[i];
        s_idx[i] = (e >= 0 && e < E) ? (int)e : -1;
    }
    __syncthreads();

    if (do_send && is_tail_cta) {
        // ---- count all-gather: my E counts go to every rank ----
        for (int i = tid; i < E; i += kLLThreads) s_hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < T * K; i += kLLThreads)
            if (s_idx[i] >= 0) atomicAdd(&s_hist[s_idx[i]], 1);
        __syncthreads();
        for (int i = tid; i < E * R; i += kLLThreads) {
            const int d = i / E, e = i % E;
            if (ld_relaxed_sys(&my->ll_mask[d])) continue;
            st_relaxed_sys(c.at<int>(d, a.region.counts_off[P]) + (size_t)me * E + e, s_hist[e]);
        }
        __syncthreads();
        if (tid < R && !ld_relaxed_sys(&my->ll_mask[tid])) {
            fence_acq_rel_sys();
            st_release_sys(&c.ctrl(tid)->ll_count_seq[P][me], seq);
        }
    }

    if (do_send && !is_tail_cta) {
        for (int t = blockIdx.x; t < T; t += num_token_ctas) {
            // slot of selection (t,k) among this rank's earlier selections of the same expert
            for (int k = warp; k < K; k += kLLWarps) {
                const int e = s_idx[t * K + k];
                int n = 0;
                if (e >= 0)
                    for (int i = lane; i < t * K + k; i += 32) n += (s_idx[i] == e) ? 1 : 0;
                n = warp_sum(n);
                if (lane == 0) {
                    s_row[k] = e >= 0 ? n : -1;
                    s_dst_rank[k] = e >= 0 ? e / L : 0;
                    s_dst_le[k] = e >= 0 ? e % L : 0;
                    if (a.send_slot != nullptr) a.send_slot[t * K + k] = e >= 0 ? n : -1;
                }
            }
            // counts of the ranks before me decide where my segment starts
            if (tid < me && !ld_relaxed_sys(&my->ll_mask[tid])) {
                const long long t0 = clock64();
                if (!wait_ge_sys(&my->ll_count_seq[P][tid], seq, c.timeout_cycles)) {
                    report(c.status, kTimeoutLLCount, me, tid, 0);
                    s_ok = 0;
                }
                if (a.wait_cost_stats != nullptr && blockIdx.x == 0) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
            }
            __syncthreads();
            if (!s_ok) return;
            if (tid < K && s_row[tid] >= 0) {
                const int e = s_dst_rank[tid] * L + s_dst_le[tid];
                int begin = 0;
                for (int src = 0; src < me; ++src)
                    if (!ld_relaxed_sys(&my->ll_mask[src])) begin += ld_relaxed_sys(&my_counts[(size_t)src * E + e]);
                const int row = begin + s_row[tid];
                const bool masked = ld_relaxed_sys(&my->ll_mask[s_dst_rank[tid]]) != 0;
                if (row >= N || masked) s_row[tid] = -1;  // cannot happen with a consistent max_tokens
                else {
                    s_row[tid] = row;
                    atomicAdd(&s_sent[s_dst_rank[tid]], 1);
                }
            }
            __syncthreads();

            if (a.use_fp8) {
                const char* src = reinterpret_cast<const char*>(a.x) + (size_t)t * H * 2;
                const int num_scales = H / 128;
                for (int c0 = 0; c0 < H; c0 += kLLThreads * 16) {
                    const int ch = c0 + tid * 16;
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
                    fp8_scale_from_amax(amax, a.round_scale != 0 || a.use_ue8m0 != 0, scale, inv);
                    int4 q;
                    q.x = (int)pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                    q.y = (int)pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                    q.z = (int)pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                    q.w = (int)pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                    uint32_t packed_exp = 0;
                    if (a.use_ue8m0) {
                        const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
                        packed_exp = __shfl_sync(0xffffffffu, ex, 0) | (__shfl_sync(0xffffffffu, ex, 8) << 8) |
                                     (__shfl_sync(0xffffffffu, ex, 16) << 16) | (__shfl_sync(0xffffffffu, ex, 24) << 24);
                    }
                    if (!act) continue;
                    for (int k = 0; k < K; ++k) {
                        const int row = s_row[k];
                        if (row < 0) continue;
                        const int d = s_dst_rank[k];
                        const size_t slot = (size_t)s_dst_le[k] * N + row;
                        st_stream(reinterpret_cast<int4*>(c.at<char>(d, a.region.recv_x_off[P]) + slot * H + ch), q);
                        if (a.use_ue8m0) {
                            if (lane == 0) c.at<uint32_t>(d, a.region.recv_scales_off[P])[slot * (H / 512) + (ch >> 9)] = packed_exp;
                        } else if ((lane & 7) == 0) {
                            c.at<float>(d, a.region.recv_scales_off[P])[slot * num_scales + (ch >> 7)] = scale;
                        }
                    }
                }
            } else {
                const int n16 = H / 8;
                const int4* src = reinterpret_cast<const int4*>(a.x) + (size_t)t * n16;
                for (int i = tid; i < n16; i += kLLThreads) {
                    const int4 v = ld_cached(src + i);
                    for (int k = 0; k < K; ++k) {
                        const int row = s_row[k];
                        if (row < 0) continue;
                        const size_t slot = (size_t)s_dst_le[k] * N + row;
                        st_stream(reinterpret_cast<int4*>(c.at<char>(s_dst_rank[k], a.region.recv_x_off[P])) + slot * n16 + i, v);
                    }
                }
            }
            if (tid < K && s_row[tid] >= 0)
                c.at<int>(s_dst_rank[tid], a.region.recv_src_info_off[P])[(size_t)s_dst_le[tid] * N + s_row[tid]] = t;
            __syncthreads();
        }
        // one release reduction per destination rank for everything this CTA sent
        if (tid < R && s_sent[tid] > 0) {
            fence_acq_rel_sys();
            red_add_release_sys(&c.ctrl(tid)->ll_data_arrived[P][me], (uint64_t)s_sent[tid]);
        }
    }

    if (do_recv && is_tail_cta) {
        // ---- receive side: counts -> layout, then wait for the rows ----
        if (tid < R && !ld_relaxed_sys(&my->ll_mask[tid])) {
            const long long t0 = clock64();
            if (!wait_ge_sys(&my->ll_count_seq[P][tid], seq, c.timeout_cycles)) {
                report(c.status, kTimeoutLLCount, me, tid, 1);
                if (c.mask_on_timeout) st_relaxed_sys(&my->ll_mask[tid], 1);
                else s_ok = 0;
            }
            if (a.wait_cost_stats != nullptr) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
        }
        __syncthreads();
        if (!s_ok) return;
        __shared__ int s_expected[kMaxRanks];
        if (tid < kMaxRanks) s_expected[tid] = 0;
        __syncthreads();
        for (int le = tid; le < L; le += kLLThreads) {
            int run = 0;
            for (int src = 0; src < R; ++src) {
                const int cnt = ld_relaxed_sys(&my->ll_mask[src]) ? 0 : ld_relaxed_sys(&my_counts[(size_t)src * E + me * L + le]);
                a.layout_range[(size_t)le * R + src] = ((int64_t)run << 32) | (int64_t)cnt;
                run += cnt;
                if (cnt) atomicAdd(&s_expected[src], cnt);
            }
            a.packed_recv_count[le] = run;
            if (a.cumulative_stats != nullptr) a.cumulative_stats[le] += run;
        }
        __syncthreads();
        if (tid < R && !ld_relaxed_sys(&my->ll_mask[tid])) {
            uint64_t* ew = expected_word(c, 0, P, tid);
            const uint64_t want = *ew + (uint64_t)s_expected[tid];
            const long long t0 = clock64();
            if (!wait_ge_sys(&my->ll_data_arrived[P][tid], want, c.timeout_cycles)) {
                report(c.status, kTimeoutLLData, me, tid, 0);
                if (c.mask_on_timeout) st_relaxed_sys(&my->ll_mask[tid], 1);
            }
            if (a.wait_cost_stats != nullptr) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
            *ew = want;
        }
    }

    if (do_recv) {
        if (cta_is_last(c.local_scratch + kTicketLLDispatch, gridDim.x) && tid == 0) commit_seq(c, kFamLLDispatch, seq);
    }
}

cudaError_t launch_ll_dispatch(const LLDispatchArgs* a, int nv, cudaStream_t stream) {
    const size_t smem = ((size_t)a[0].num_tokens * a[0].num_topk + a[0].num_experts) * sizeof(int);
    return DX_LAUNCH_RANKED(ll_dispatch_kernel, LLDispatchArgs, a, nv, a[0].num_sms, kLLThreads, smem, stream);
}

// =============================================================================================
// combine
// =============================================================================================
template <int V>
__global__ void __launch_bounds__(kLLThreads, 1) ll_combine_kernel(const __grid_constant__ ArgPack<LLCombineArgs, V> pack) {
    const LLCombineArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk, E = a.num_experts;
    const int L = E / R, H = a.hidden, P = a.parity;
    const int N = R * a.num_max_tokens, M = a.num_max_tokens;
    const int n16 = H / 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t seq = next_seq(c, kFamLLCombine);
    const bool do_send = a.phases & 1, do_recv = a.phases & 2;
    ControlBlock* my = c.my_ctrl();
    __shared__ int s_sent[kMaxRanks];
    __shared__ int s_expected[kMaxRanks];
    __shared__ int s_ok;
    if (tid < kMaxRanks) {
        s_sent[tid] = 0;
        s_expected[tid] = 0;
    }
    if (tid == 0) s_ok = 1;
    __syncthreads();

    if (do_send) {
        // every valid (local expert, slot) row goes back to the rank it came from
        const int total_warps = gridDim.x * kLLWarps;
        for (int s = blockIdx.x * kLLWarps + warp; s < L * N; s += total_warps) {
            const int le = s / N, n = s % N;
            int64_t lr = (lane < R) ? a.layout_range[(size_t)le * R + lane] : 0;
            const int begin = (int)(lr >> 32), cnt = (int)(lr & 0xffffffff);
            const unsigned hit = __ballot_sync(0xffffffffu, lane < R && n >= begin && n < begin + cnt);
            if (hit == 0) continue;
            const int src = __ffs(hit) - 1;
            if (ld_relaxed_sys(&my->ll_mask[src])) continue;
            const int token = a.src_info[(size_t)le * N + n];
            if (token < 0 || token >= M) continue;
            const int4* from = reinterpret_cast<const int4*>(a.x) + (size_t)s * n16;
            int4* to = reinterpret_cast<int4*>(c.at<char>(src, a.region.combine_stage_off[P])) +
                       ((size_t)(me * L + le) * M + token) * n16;
            constexpr int U = 4;
            for (int i0 = 0; i0 < n16; i0 += 32 * U) {
                int4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    if (i < n16) v[u] = ld_stream(from + i);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    if (i < n16) st_stream(to + i, v[u]);
                }
            }
            if (lane == 0) atomicAdd(&s_sent[src], 1);
        }
        __syncthreads();
        if (tid < R && s_sent[tid] > 0) {
            fence_acq_rel_sys();
            red_add_release_sys(&c.ctrl(tid)->ll_combine_arrived[P][me], (uint64_t)s_sent[tid]);
        }
    }

    if (do_recv) {
        // rows I expect from every rank = my valid selections that live there
        for (int i = tid; i < T * K; i += kLLThreads) {
            const int64_t e = a.topk_idx[i];
            if (e >= 0 && e < E) atomicAdd(&s_expected[(int)e / L], 1);
        }
        __syncthreads();
        if (tid < R && !ld_relaxed_sys(&my->ll_mask[tid])) {
            const uint64_t want = *expected_word(c, 1, P, tid) + (uint64_t)s_expected[tid];
            const long long t0 = clock64();
            if (!wait_ge_sys(&my->ll_combine_arrived[P][tid], want, c.timeout_cycles)) {
                report(c.status, kTimeoutCombineData, me, tid, 0);
                if (c.mask_on_timeout) st_relaxed_sys(&my->ll_mask[tid], 1);
                else s_ok = 0;
            }
            if (a.wait_cost_stats != nullptr && blockIdx.x == 0) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
        }
        __syncthreads();
        if (s_ok) {
            const int4* stage = reinterpret_cast<const int4*>(c.at<char>(me, a.region.combine_stage_off[P]));
            __shared__ long long s_sel_row[kMaxTopk];  // stage row of selection k, -1 = skip
            __shared__ float s_sel_w[kMaxTopk];
            for (int t = blockIdx.x; t < T; t += gridDim.x) {
                __syncthreads();
                if (tid < K) {
                    const int64_t e = a.topk_idx[(size_t)t * K + tid];
                    const bool ok = e >= 0 && e < E && !ld_relaxed_sys(&my->ll_mask[(int)e / L]);
                    s_sel_row[tid] = ok ? ((long long)e * M + t) * n16 : -1;
                    s_sel_w[tid] = ok ? a.topk_weights[(size_t)t * K + tid] : 0.f;
                }
                __syncthreads();
                for (int i = tid; i < n16; i += kLLThreads) {
                    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    for (int k0 = 0; k0 < K; k0 += 8) {
                        int4 v[8];
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const long long row = k < K ? s_sel_row[k] : -1;
                            v[kk] = row >= 0 ? ld_peer(stage + row + i) : make_int4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const float w = k < K ? s_sel_w[k] : 0.f;
                            const uint32_t u[4] = {(uint32_t)v[kk].x, (uint32_t)v[kk].y, (uint32_t)v[kk].z, (uint32_t)v[kk].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 p = bf16x2_to_f2(u[j]);
                                acc[2 * j] = fmaf(w, p.x, acc[2 * j]);
                                acc[2 * j + 1] = fmaf(w, p.y, acc[2 * j + 1]);
                            }
                        }
                    }
                    int4 o;
                    o.x = (int)f2_to_bf16x2(acc[0], acc[1]);
                    o.y = (int)f2_to_bf16x2(acc[2], acc[3]);
                    o.z = (int)f2_to_bf16x2(acc[4], acc[5]);
                    o.w = (int)f2_to_bf16x2(acc[6], acc[7]);
                    st_stream(reinterpret_cast<int4*>(a.out) + (size_t)t * n16 + i, o);
                }
            }
        }
        if (cta_is_last(c.local_scratch + kTicketLLCombine, gridDim.x)) {
            if (tid < R) *expected_word(c, 1, P, tid) += (uint64_t)s_expected[tid];
            if (tid == 0) commit_seq(c, kFamLLCombine, seq);
        }
    }
}

cudaError_t launch_ll_combine(const LLCombineArgs* a, int nv, cudaStream_t stream) {
    return DX_LAUNCH_RANKED(ll_combine_kernel, LLCombineArgs, a, nv, a[0].num_sms, kLLThreads, 0, stream);
}

}  // namespace dx
