// Low-latency dispatch / combine for ~128 tokens per rank over one NVSwitch domain.
//
// dispatch (one launch):
//   * every rank all-gathers its per-expert selection counts (E words per peer; every word carries a validity tag of the
//     call, so there is no flag and no release behind them, and a receiver polls exactly the words it uses),
//   * one CTA per token quantises the row in registers (BF16 -> e4m3, one scale per 128 channels) while
//     the counts are in flight, then stores it K times straight into the FINAL position of the peers'
//     packed_recv_x: row `sum_{src<me} count[src][e] + slot` of expert e, which every sender can compute
//     from the all-gathered counts. There is no send buffer, no receive-side unpack pass and no memset
//     of the [L, N, hidden] output,
//   * arrival is counted per source rank with monotonic release reductions; the last CTA derives
//     packed_recv_count / layout_range from the counts and waits for the rows.
// combine (one launch), two forms chosen by where the expert outputs live:
//   * pull (outputs in symmetric memory: the zero-copy buffer or an arena tensor): every rank posts "my outputs are
//     final, at this offset" to all home ranks; one CTA per token then loads the token's K rows straight from the
//     peers (their position was recorded by dispatch), does sum_k w[t,k] * row in fp32 registers and writes BF16 once.
//     No stage buffer, no second pass, one self-validating word per peer. When it directly follows the dispatch of its
//     handle it overlaps that kernel's wait for the last rows (see combine_pull);
//   * push (outputs in ordinary device memory): expert ranks push their BF16 rows into the home rank's
//     [E][max_tokens] stage (address = (expert, token), so no metadata travels), the home rank waits per source,
//     then reduces as above.
//   Both are deterministic (fixed k order, no atomics) and may write the result to pinned host memory.
//
// `phases` splits either kernel into its send (bit 0) and receive (bit 1) half for the
// return_recv_hook contract. Sequence numbers and expected-arrival totals live on the device, so a
// launch carries no per-call value besides the buffer parity.
//
// Cost model that shaped the code (measured with the trace stamps on B200): a system-scope release
// costs 1-6 us when many stores are outstanding, so each CTA issues exactly one per destination rank
// and all CTA-local bookkeeping uses GPU scope; every same-address shared-memory atomic serialises, so
// counts are warp-aggregated.
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

struct QuantChunk {
    int4 q;
    float scale;
    uint32_t packed_exp;
};

// BF16 -> e4m3 for the 16 channels [ch, ch+16) of a row; 8 lanes share a scale, a warp covers four.
__device__ __forceinline__ QuantChunk quantize_chunk(const char* row, int ch, bool act, bool pow2, bool ue8m0) {
    int4 r0 = make_int4(0, 0, 0, 0), r1 = r0;
    if (act) {
        r0 = ld_cached(reinterpret_cast<const int4*>(row + (size_t)ch * 2));
        r1 = ld_cached(reinterpret_cast<const int4*>(row + (size_t)ch * 2 + 16));
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
    float inv;
    QuantChunk o;
    fp8_scale_from_amax(amax, pow2, o.scale, inv);
    o.q.x = (int)pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
    o.q.y = (int)pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
    o.q.z = (int)pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
    o.q.w = (int)pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
    o.packed_exp = 0;
    if (ue8m0) {
        const uint32_t ex = (__float_as_uint(o.scale) >> 23) & 0xffu;
        o.packed_exp = __shfl_sync(0xffffffffu, ex, 0) | (__shfl_sync(0xffffffffu, ex, 8) << 8) |
                       (__shfl_sync(0xffffffffu, ex, 16) << 16) | (__shfl_sync(0xffffffffu, ex, 24) << 24);
    }
    return o;
}

// =============================================================================================
// dispatch
// =============================================================================================
// The kernels are named dx::ll::dispatch and dx::ll::combine: tools written for the reference and for upstream DeepEP
// (tests/utils.py:173-271) find the low-latency kernels in a profiler trace by the substrings "::dispatch" / "::combine".
// A count word carries its own validity tag, (tag << 16) | count with tag = (sequence mod 65535) + 1, so the sender needs no
// release behind the counts and a receiver polls exactly the words it uses. A parity's matrix is rewritten every second call, so a
// stale word never carries the current tag; the matrices start zeroed (tag 0 is never used).
__device__ __forceinline__ int ll_count_tag(uint64_t seq) { return (int)(seq % 65535ull) + 1; }

// Bounded poll of one count word: the count, or -1 when the limit ran out.
__device__ __forceinline__ int wait_tagged_count(const int* p, int tag, long long limit) {
    unsigned w = (unsigned)ld_relaxed_sys(p);
    if ((w >> 16) == (unsigned)tag) return (int)(w & 0xffffu);
    const long long t0 = clock64();
    while (((w = (unsigned)ld_relaxed_sys(p)) >> 16) != (unsigned)tag) {
        if (clock64() - t0 > limit) return -1;
    }
    return (int)(w & 0xffffu);
}

namespace ll {
template <int V>
__global__ void __launch_bounds__(kLLThreads, 1) dispatch(const __grid_constant__ ArgPack<LLDispatchArgs, V> pack) {
    pdl_wait_predecessor();
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
    int* s_hist = s_mem + T * K;     // [E] tail CTA: my counts per expert; token CTAs: selections per expert among earlier tokens
    __shared__ int s_ok;
    __shared__ int s_mask[kMaxRanks];
    __shared__ int s_row[kMaxTopk];      // destination row inside the expert, -1 = skip
    __shared__ int s_dst_rank[kMaxTopk];
    __shared__ int s_dst_le[kMaxTopk];
    __shared__ int s_sent[kMaxRanks];
    __shared__ int s_expected[kMaxRanks];
    __shared__ int s_cnt[kMaxTopk][kMaxRanks];  // counts of the ranks before me for the experts of the current token
    const int count_tag = ll_count_tag(seq);

    // Which call last used this parity: a combine that the stream lets start while this kernel still waits for its last rows
    // (programmatic dependent launch) learns from it that its dispatch is in flight, and what tag the row numbers carry.
    // Written (and fenced) before this CTA allows the successor's launch, so no successor CTA can run before it is in memory.
    if (do_send && blockIdx.x == 0 && tid == 0) {
        *reinterpret_cast<volatile uint64_t*>(c.seq + kLLStartedWord0 + P) = seq;
        __threadfence();
    }
    __syncthreads();
    pdl_release_successor();
    const int tslot = is_tail_cta ? 1 : 0;
    const bool traced = is_tail_cta || blockIdx.x == 0;
    if (traced) trace_stamp(c, kFamLLDispatch, tslot, 0);
    if (tid == 0) s_ok = 1;
    if (tid < kMaxRanks) {
        s_sent[tid] = 0;
        s_expected[tid] = 0;
        s_mask[tid] = tid < R ? __ldcg(&my->ll_mask[tid]) : 1;
    }
    for (int i = tid; i < T * K; i += kLLThreads) {
        const int64_t e = a.topk_idx[i];
        s_idx[i] = (e >= 0 && e < E) ? (int)e : -1;
    }
    __syncthreads();
    if (traced) trace_stamp(c, kFamLLDispatch, tslot, 1);

    if (do_send && is_tail_cta) {
        // ---- count all-gather: my E counts go to every rank, then ONE release per rank ----
        for (int i = tid; i < E; i += kLLThreads) s_hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < T * K; i += kLLThreads)
            if (s_idx[i] >= 0) atomicAdd(&s_hist[s_idx[i]], 1);
        __syncthreads();
        const int tagw = count_tag << 16;
        if ((E & 3) == 0) {
            const int e4 = E / 4;
            for (int i = tid; i < e4 * R; i += kLLThreads) {
                const int d = i / e4, j = i % e4;
                if (s_mask[d]) continue;
                const int4 v = make_int4(tagw | s_hist[4 * j], tagw | s_hist[4 * j + 1], tagw | s_hist[4 * j + 2], tagw | s_hist[4 * j + 3]);
                *(reinterpret_cast<int4*>(c.at<int>(d, a.region.counts_off[P]) + (size_t)me * E) + j) = v;
            }
        } else {
            for (int i = tid; i < E * R; i += kLLThreads) {
                const int d = i / E, e = i % E;
                if (!s_mask[d]) c.at<int>(d, a.region.counts_off[P])[(size_t)me * E + e] = tagw | s_hist[e];
            }
        }
        // no release: every word says for itself whether it belongs to this call
        trace_stamp(c, kFamLLDispatch, 1, 2);
    }

    if (do_send && !is_tail_cta) {
        const bool pow2 = a.round_scale != 0 || a.use_ue8m0 != 0;
        // s_hist[e] = selections of expert e among the tokens before `hist_upto`; tokens are visited in rising order, so
        // the running histogram is advanced instead of rescanning all earlier selections for every token
        for (int i = tid; i < E; i += kLLThreads) s_hist[i] = 0;
        int hist_upto = 0;
        bool counts_known = false;
        __syncthreads();
        for (int t = blockIdx.x; t < T; t += num_token_ctas) {
            // First chunk of the row is quantised while the counts of the other ranks are still in flight.
            const char* xrow = reinterpret_cast<const char*>(a.x) + (size_t)t * H * 2;
            QuantChunk qc;
            const bool act0 = tid * 16 < H;
            if (a.use_fp8) qc = quantize_chunk(xrow, tid * 16, act0, pow2, a.use_ue8m0 != 0);
            for (int i = hist_upto * K + tid; i < t * K; i += kLLThreads)
                if (s_idx[i] >= 0) atomicAdd(&s_hist[s_idx[i]], 1);
            hist_upto = t;
            __syncthreads();
            // slot of selection (t,k) among this rank's earlier selections of the same expert
            if (tid < K) {
                const int e = s_idx[t * K + tid];
                int n = -1;
                if (e >= 0) {
                    n = s_hist[e];
                    for (int k2 = 0; k2 < tid; ++k2) n += (s_idx[t * K + k2] == e) ? 1 : 0;
                }
                s_row[tid] = n;
                s_dst_rank[tid] = e >= 0 ? e / L : 0;
                s_dst_le[tid] = e >= 0 ? e % L : 0;
            }
            __syncthreads();
            // counts of the ranks before me decide where my segment starts: one thread per (selection, lower rank) polls its word
            for (int i = tid; i < K * me; i += kLLThreads) {
                const int k = i / me, src = i % me;
                int cnt = 0;
                if (s_row[k] >= 0 && !s_mask[src]) {
                    const long long t0 = clock64();
                    cnt = wait_tagged_count(&my_counts[(size_t)src * E + s_dst_rank[k] * L + s_dst_le[k]], count_tag, c.timeout_cycles);
                    if (cnt < 0) {
                        cnt = 0;
                        report(c.status, kTimeoutLLCount, me, src, 0);
                        if (c.mask_on_timeout) {
                            // shrink mode: a silent rank sends nothing to anybody, so every sender drops its counts alike
                            st_relaxed_sys(&my->ll_mask[src], 1);
                            s_mask[src] = 1;
                        } else {
                            s_ok = 0;
                        }
                    }
                    if (a.wait_cost_stats != nullptr && blockIdx.x == 0 && k == 0 && !counts_known)
                        atomicAdd((unsigned long long*)&a.wait_cost_stats[src], (unsigned long long)(clock64() - t0));
                }
                s_cnt[k][src] = cnt;
            }
            counts_known = true;
            __syncthreads();
            if (!s_ok) break;  // falls through to the completion ticket; nothing was sent by this CTA
            if (traced) trace_stamp(c, kFamLLDispatch, 0, 2);
            if (tid < K) {
                int final_row = -1;
                if (s_row[tid] >= 0) {
                    const int e = s_dst_rank[tid] * L + s_dst_le[tid];
                    int begin = 0;
                    for (int src = 0; src < me; ++src)
                        if (!s_mask[src]) begin += s_cnt[tid][src];
                    const int row = begin + s_row[tid];
                    const size_t row_bytes = (size_t)H * (a.use_fp8 ? 1 : 2);
                    if (row >= N || s_mask[s_dst_rank[tid]] ||
                        !peer_range_ok(c, s_dst_rank[tid], c.at<char>(s_dst_rank[tid], a.region.recv_x_off[P]) + ((size_t)s_dst_le[tid] * N + (row < N ? row : 0)) * row_bytes, row_bytes, 3)) {
                        s_row[tid] = -1;  // row >= N cannot happen with a consistent max_tokens
                    } else {
                        s_row[tid] = row;
                        final_row = row;
                        atomicAdd(&s_sent[s_dst_rank[tid]], 1);
                    }
                }
                // where this selection landed at its expert's rank: the pull form of combine reads the output row back from there
                // (tagged like the count words: a combine that overlaps this kernel polls the word until it is this call's)
                if (a.send_row != nullptr) a.send_row[t * K + tid] = (count_tag << 16) | (final_row + 1);
            }
            __syncthreads();
            if (traced) trace_stamp(c, kFamLLDispatch, 0, 3);

            if (a.use_fp8) {
                const int num_scales = H / 128;
                for (int c0 = 0; c0 < H; c0 += kLLThreads * 16) {
                    const int ch = c0 + tid * 16;
                    const bool act = ch < H;
                    if (c0 > 0) qc = quantize_chunk(xrow, ch, act, pow2, a.use_ue8m0 != 0);
                    if (!act) continue;
                    for (int k = 0; k < K; ++k) {
                        const int row = s_row[k];
                        if (row < 0) continue;
                        const int d = s_dst_rank[k];
                        const size_t slot = (size_t)s_dst_le[k] * N + row;
                        st_stream(reinterpret_cast<int4*>(c.at<char>(d, a.region.recv_x_off[P]) + slot * H + ch), qc.q);
                        if (a.use_ue8m0) {
                            if (lane == 0) c.at<uint32_t>(d, a.region.recv_scales_off[P])[slot * (H / 512) + (ch >> 9)] = qc.packed_exp;
                        } else if ((lane & 7) == 0) {
                            c.at<float>(d, a.region.recv_scales_off[P])[slot * num_scales + (ch >> 7)] = qc.scale;
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
            if (traced) trace_stamp(c, kFamLLDispatch, 0, 4);
        }
        // one release reduction per destination rank for everything this CTA sent
        if (tid < R && s_sent[tid] > 0) red_add_release_sys(&c.ctrl(tid)->ll_data_arrived[P][me], (uint64_t)s_sent[tid]);
        if (traced) trace_stamp(c, kFamLLDispatch, 0, 5);
    }

    if (do_recv && is_tail_cta) {
        // ---- receive side: counts -> layout, then wait for the rows ----
        __syncthreads();  // the send part is done with s_hist: from here on it holds the counts received, [R][L]
        for (int i = tid; i < R * L; i += kLLThreads) {
            const int src = i / L, le = i % L;
            int cnt = 0;
            if (!s_mask[src]) {
                const long long t0 = clock64();
                cnt = wait_tagged_count(&my_counts[(size_t)src * E + me * L + le], count_tag, c.timeout_cycles);
                if (cnt < 0) {
                    cnt = 0;
                    report(c.status, kTimeoutLLCount, me, src, 1);
                    if (c.mask_on_timeout) {
                        st_relaxed_sys(&my->ll_mask[src], 1);
                        s_mask[src] = 1;
                    } else {
                        s_ok = 0;
                    }
                }
                if (a.wait_cost_stats != nullptr && le == 0) atomicAdd((unsigned long long*)&a.wait_cost_stats[src], (unsigned long long)(clock64() - t0));
            }
            s_hist[i] = cnt;
        }
        __syncthreads();
        trace_stamp(c, kFamLLDispatch, 1, 3);
        const bool counts_ok = s_ok != 0;  // a failed count wait (without shrink mode) skips the layout, never the completion ticket
        for (int le = tid; counts_ok && le < L; le += kLLThreads) {
            int run = 0;
            for (int src = 0; src < R; ++src) {
                const int cnt = s_mask[src] ? 0 : s_hist[src * L + le];
                a.layout_range[(size_t)le * R + src] = ((int64_t)run << 32) | (int64_t)cnt;
                run += cnt;
            }
            a.packed_recv_count[le] = run;
            if (a.cumulative_stats != nullptr) a.cumulative_stats[le] += run;
        }
        // rows expected from every source: one warp per source sums its L counts
        for (int src = warp; counts_ok && src < R; src += kLLWarps) {
            int sum = 0;
            if (!s_mask[src])
                for (int le = lane; le < L; le += 32) sum += s_hist[src * L + le];
            sum = warp_sum(sum);
            if (lane == 0) s_expected[src] = sum;
        }
        __syncthreads();
        trace_stamp(c, kFamLLDispatch, 1, 4);
        if (counts_ok && tid < R && !s_mask[tid]) {
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
        trace_stamp(c, kFamLLDispatch, 1, 5);
    }

    if (do_recv) {
        if (cta_is_last(c.local_scratch + kTicketLLDispatch, gridDim.x) && tid == 0) commit_seq(c, kFamLLDispatch, seq);
        if (traced) trace_stamp(c, kFamLLDispatch, tslot, 6);
    }
}

}  // namespace ll

cudaError_t launch_ll_dispatch(const LLDispatchArgs* a, int nv, cudaStream_t stream) {
    const size_t smem = ((size_t)a[0].num_tokens * a[0].num_topk + a[0].num_experts) * sizeof(int);
    return DX_LAUNCH_RANKED_PDL(ll::dispatch, LLDispatchArgs, a, nv, a[0].num_sms, kLLThreads, smem, stream);
}

// =============================================================================================
// combine
// =============================================================================================
namespace ll {
template <int V>
__global__ void __launch_bounds__(kLLThreads, 1) combine(const __grid_constant__ ArgPack<LLCombineArgs, V> pack) {
    pdl_wait_predecessor();
    pdl_release_successor();
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
    extern __shared__ int s_cum[];  // [L+1] exclusive prefix of valid rows per local expert
    __shared__ int s_mask[kMaxRanks];
    __shared__ int s_sent[kMaxRanks];
    __shared__ int s_expected[kMaxRanks];
    __shared__ int s_ok;
    if (tid < kMaxRanks) {
        s_sent[tid] = 0;
        s_expected[tid] = 0;
        s_mask[tid] = tid < R ? __ldcg(&my->ll_mask[tid]) : 1;
    }
    if (tid == 0) s_ok = 1;
    const bool traced = blockIdx.x == 0 || blockIdx.x == gridDim.x - 1;
    const int tslot = blockIdx.x == 0 ? 0 : 1;
    if (traced) trace_stamp(c, kFamLLCombine, tslot, 0);
    __syncthreads();
    if (do_recv) {
        // rows I expect from every rank = my valid selections that live there (warp-aggregated count); done first so
        // that it does not sit between the last arriving row and the reduction
        for (int i0 = 0; i0 < T * K; i0 += kLLThreads) {
            const int i = i0 + tid;
            int rk = -1;
            if (i < T * K) {
                const int64_t e = a.topk_idx[i];
                if (e >= 0 && e < E) rk = (int)e / L;
            }
            for (int r = 0; r < R; ++r) {
                const unsigned b = __ballot_sync(0xffffffffu, rk == r);
                if (lane == 0 && b) atomicAdd(&s_expected[r], __popc(b));
            }
        }
        __syncthreads();
    }

    if (do_send) {
        // ---- enumerate the valid rows compactly: row r -> (local expert, slot) through a prefix over experts ----
        for (int le = tid; le < L; le += kLLThreads) {
            int cnt = 0;
            for (int src = 0; src < R; ++src) cnt += (int)(a.layout_range[(size_t)le * R + src] & 0xffffffff);
            s_cum[le + 1] = cnt;
        }
        if (tid == 0) s_cum[0] = 0;
        __syncthreads();
        if (warp == 0) {
            // inclusive scan of s_cum[1..L] by one warp, each lane owning a contiguous chunk
            const int per = (L + 31) / 32;
            const int b = 1 + lane * per, e = min(1 + L, b + per);
            int sum = 0;
            for (int i = b; i < e; ++i) sum += s_cum[i];
            const int incl = warp_incl_scan(sum);
            int run = incl - sum;
            for (int i = b; i < e; ++i) {
                run += s_cum[i];
                s_cum[i] = run;
            }
        }
        __syncthreads();
        const int total_rows = s_cum[L];
        const int total_warps = gridDim.x * kLLWarps;
        // two warps per row (each copies half of it with all of its loads in flight at once)
        const int half16 = (n16 + 1) / 2;
        for (int item = blockIdx.x * kLLWarps + warp; item < 2 * total_rows; item += total_warps) {
            const int r = item >> 1, part = item & 1;
            // largest le with s_cum[le] <= r
            int lo = 0, hi = L;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_cum[mid] <= r) lo = mid;
                else hi = mid;
            }
            const int le = lo, n = r - s_cum[le];
            const int64_t lr = (lane < R) ? a.layout_range[(size_t)le * R + lane] : 0;
            const int begin = (int)(lr >> 32), cnt = (int)(lr & 0xffffffff);
            const unsigned hit = __ballot_sync(0xffffffffu, lane < R && n >= begin && n < begin + cnt);
            if (hit == 0) continue;
            const int src = __ffs(hit) - 1;
            if (s_mask[src]) continue;
            const int token = a.src_info[(size_t)le * N + n];
            if (token < 0 || token >= M) continue;
            const int4* from = reinterpret_cast<const int4*>(a.x) + ((size_t)le * N + n) * n16;
            int4* to = reinterpret_cast<int4*>(c.at<char>(src, a.region.combine_stage_off[P])) + ((size_t)(me * L + le) * M + token) * n16;
            if (!peer_range_ok(c, src, to, (size_t)n16 * 16, 4)) continue;
            const int lo16 = part * half16, hi16 = min(n16, lo16 + half16);
            constexpr int U = 14;
            for (int i0 = lo16; i0 < hi16; i0 += 32 * U) {
                int4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    if (i < hi16) v[u] = ld_stream(from + i);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    if (i < hi16) st_stream(to + i, v[u]);
                }
            }
            if (lane == 0 && part == 0) atomicAdd(&s_sent[src], 1);
        }
        __syncthreads();
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 1);
        if (tid < R && s_sent[tid] > 0) red_add_release_sys(&c.ctrl(tid)->ll_combine_arrived[P][me], (uint64_t)s_sent[tid]);
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 2);
    }

    if (do_recv) {
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 3);
        if (tid < R && !s_mask[tid]) {
            const uint64_t want = *expected_word(c, 1, P, tid) + (uint64_t)s_expected[tid];
            const long long t0 = clock64();
            if (!wait_ge_sys(&my->ll_combine_arrived[P][tid], want, c.timeout_cycles)) {
                report(c.status, kTimeoutCombineData, me, tid, 0);
                if (c.mask_on_timeout) {
                    st_relaxed_sys(&my->ll_mask[tid], 1);
                    s_mask[tid] = 1;
                } else {
                    s_ok = 0;
                }
            }
            if (a.wait_cost_stats != nullptr && blockIdx.x == 0) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
        }
        __syncthreads();
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 4);
        if (s_ok) {
            const int4* stage = reinterpret_cast<const int4*>(c.at<char>(me, a.region.combine_stage_off[P]));
            __shared__ long long s_sel_row[kMaxTopk];  // stage row of selection k, -1 = skip
            __shared__ float s_sel_w[kMaxTopk];
            for (int t = blockIdx.x; t < T; t += gridDim.x) {
                __syncthreads();
                if (tid < K) {
                    const int64_t e = a.topk_idx[(size_t)t * K + tid];
                    const bool ok = e >= 0 && e < E && !s_mask[(int)e / L];
                    s_sel_row[tid] = ok ? ((long long)e * M + t) * n16 : -1;
                    s_sel_w[tid] = ok ? a.topk_weights[(size_t)t * K + tid] : 0.f;
                }
                __syncthreads();
                // two 16-byte columns per thread per pass, all loads of a pass in flight together
                for (int i0 = 0; i0 < n16; i0 += 2 * kLLThreads) {
                    const int ia = i0 + tid, ib = i0 + kLLThreads + tid;
                    float acc[2][8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[0][j] = acc[1][j] = 0.f;
                    for (int k0 = 0; k0 < K; k0 += 8) {
                        int4 va[8], vb[8];
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const long long row = k < K ? s_sel_row[k] : -1;
                            va[kk] = (row >= 0 && ia < n16) ? ld_peer(stage + row + ia) : make_int4(0, 0, 0, 0);
                            vb[kk] = (row >= 0 && ib < n16) ? ld_peer(stage + row + ib) : make_int4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const float w = k < K ? s_sel_w[k] : 0.f;
                            const uint32_t ua[4] = {(uint32_t)va[kk].x, (uint32_t)va[kk].y, (uint32_t)va[kk].z, (uint32_t)va[kk].w};
                            const uint32_t ub[4] = {(uint32_t)vb[kk].x, (uint32_t)vb[kk].y, (uint32_t)vb[kk].z, (uint32_t)vb[kk].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 pa = bf16x2_to_f2(ua[j]), pb = bf16x2_to_f2(ub[j]);
                                acc[0][2 * j] = fmaf(w, pa.x, acc[0][2 * j]);
                                acc[0][2 * j + 1] = fmaf(w, pa.y, acc[0][2 * j + 1]);
                                acc[1][2 * j] = fmaf(w, pb.x, acc[1][2 * j]);
                                acc[1][2 * j + 1] = fmaf(w, pb.y, acc[1][2 * j + 1]);
                            }
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int i = h == 0 ? ia : ib;
                        if (i >= n16) continue;
                        int4 o;
                        o.x = (int)f2_to_bf16x2(acc[h][0], acc[h][1]);
                        o.y = (int)f2_to_bf16x2(acc[h][2], acc[h][3]);
                        o.z = (int)f2_to_bf16x2(acc[h][4], acc[h][5]);
                        o.w = (int)f2_to_bf16x2(acc[h][6], acc[h][7]);
                        st_stream(reinterpret_cast<int4*>(a.out) + (size_t)t * n16 + i, o);
                    }
                }
            }
        }
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 5);
        if (cta_is_last(c.local_scratch + kTicketLLCombine, gridDim.x)) {
            if (tid < R) *expected_word(c, 1, P, tid) += (uint64_t)s_expected[tid];
            if (tid == 0) commit_seq(c, kFamLLCombine, seq);
        }
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 6);
    }
}

// Pull form: the expert outputs of every rank sit in its symmetric buffer, so the home rank reads the K rows of a token
// where dispatch put them (send_row) and reduces them in registers. The only signalling is one self-validating word per
// (expert rank, home rank): "outputs final, at this offset" (ControlBlock::ll_pull_src).
template <int V>
__global__ void __launch_bounds__(kLLThreads, 1) combine_pull(const __grid_constant__ ArgPack<LLCombineArgs, V> pack) {
    pdl_release_successor();
    const LLCombineArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk, E = a.num_experts;
    const int L = E / R, H = a.hidden;
    const int N = R * a.num_max_tokens;
    const int n16 = H / 8;
    const int tid = threadIdx.x;
    // When this kernel directly follows the dispatch of its handle, programmatic dependent launch lets its CTAs start while
    // that dispatch still waits for the last rows of the other ranks. Nothing this kernel reads depends on those rows: the
    // expert outputs were final before the dispatch began, and the row numbers it needs are written early by the dispatch's
    // token CTAs, each word tagged with the call it belongs to. So a CTA that finds its dispatch still in flight (started, not
    // yet committed) does its work first and waits for the predecessor only before it exits, which keeps the stream's order of
    // completion. In every other case (dispatch already complete: an expert GEMM ran in between, or the launch is an ordinary
    // one) the wait comes first, as for any dependent kernel. A stale read of either word can only choose the second way.
    __shared__ int s_early;
    __shared__ unsigned long long s_seq_d;
    if (tid == 0) {
        const uint64_t started = *reinterpret_cast<volatile uint64_t*>(c.seq + kLLStartedWord0 + a.parity);
        const uint64_t committed = *reinterpret_cast<volatile uint64_t*>(c.seq + kFamLLDispatch);
        s_early = committed < started ? 1 : 0;
        s_seq_d = started;
    }
    __syncthreads();
    const bool early = s_early != 0;
    if (!early) {
        pdl_wait_predecessor();
        __syncthreads();
        if (tid == 0) s_seq_d = *reinterpret_cast<volatile uint64_t*>(c.seq + kLLStartedWord0 + a.parity);
        __syncthreads();
    }
    const int row_tag = ll_count_tag(s_seq_d);
    const uint64_t seq = next_seq(c, kFamLLCombine);
    const bool do_send = a.phases & 1, do_recv = a.phases & 2;
    ControlBlock* my = c.my_ctrl();
    __shared__ int s_mask[kMaxRanks];
    __shared__ const int4* s_base[kMaxRanks];
    __shared__ int s_ok;
    __shared__ long long s_sel_row[kMaxTopk];  // element offset (in int4) of selection k inside its rank's x, -1 = skip
    __shared__ int s_sel_rank[kMaxTopk];
    __shared__ float s_sel_w[kMaxTopk];
    if (tid < kMaxRanks) s_mask[tid] = tid < R ? __ldcg(&my->ll_mask[tid]) : 1;
    if (tid == 0) s_ok = 1;
    const bool traced = blockIdx.x == 0 || blockIdx.x == gridDim.x - 1;
    const int tslot = blockIdx.x == 0 ? 0 : 1;
    if (traced) trace_stamp(c, kFamLLCombine, tslot, 0);
    __syncthreads();

    if (do_send && blockIdx.x == 0 && tid < R && !s_mask[tid]) {
        // the kernel that produced x is complete (stream order), so its writes are in this GPU's memory system
        // one self-validating word per peer: no payload-then-flag pair, so no release round trip in front of the peers' loads
        st_relaxed_sys(&c.ctrl(tid)->ll_pull_src[seq & 1][me], ((seq & 0xffffffull) << 40) | (a.x_off & ((1ull << 40) - 1)));
    }
    if (traced) trace_stamp(c, kFamLLCombine, tslot, 1);

    if (do_recv) {
        if (tid < R && !s_mask[tid]) {
            uint64_t w[1];
            const long long t0 = clock64();
            bool got = true;
            while (((w[0] = ld_relaxed_sys(&my->ll_pull_src[seq & 1][tid])) >> 40) != (seq & 0xffffffull)) {
                if (clock64() - t0 > c.timeout_cycles) {
                    got = false;
                    break;
                }
            }
            w[0] &= (1ull << 40) - 1;
            if (!got) {
                report(c.status, kTimeoutCombineReady, me, tid, 1);
                if (c.mask_on_timeout) {
                    st_relaxed_sys(&my->ll_mask[tid], 1);
                    s_mask[tid] = 1;
                } else {
                    s_ok = 0;
                }
            } else {
                s_base[tid] = c.at<const int4>(tid, w[0]);
            }
            if (a.wait_cost_stats != nullptr && blockIdx.x == 0) atomicAdd((unsigned long long*)&a.wait_cost_stats[tid], (unsigned long long)(clock64() - t0));
        }
        __syncthreads();
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 4);
        if (s_ok) {
            for (int t = blockIdx.x; t < T; t += gridDim.x) {
                __syncthreads();
                if (tid < K) {
                    const int64_t e = a.topk_idx[(size_t)t * K + tid];
                    // the word is (tag << 16) | (row + 1); while the dispatch is still running it may not have been written yet
                    unsigned wrow = (unsigned)ld_relaxed_sys(a.send_row + (size_t)t * K + tid);
                    if ((wrow >> 16) != (unsigned)row_tag) {
                        const long long t0 = clock64();
                        while (((wrow = (unsigned)ld_relaxed_sys(a.send_row + (size_t)t * K + tid)) >> 16) != (unsigned)row_tag) {
                            if (clock64() - t0 > c.timeout_cycles) {
                                report(c.status, kTimeoutCombineReady, me, me, 2);
                                wrow = 0;
                                break;
                            }
                        }
                    }
                    const int row = (int)(wrow & 0xffffu) - 1;
                    bool ok = e >= 0 && e < E && row >= 0 && row < N && !s_mask[(int)e / L];
                    const int r = ok ? (int)e / L : 0;
                    const long long off = ok ? ((long long)((int)e % L) * N + row) * n16 : -1;
                    if (ok && !peer_range_ok(c, r, s_base[r] + off, (size_t)n16 * 16, 5)) ok = false;
                    s_sel_row[tid] = ok ? off : -1;
                    s_sel_rank[tid] = r;
                    s_sel_w[tid] = ok ? a.topk_weights[(size_t)t * K + tid] : 0.f;
                }
                __syncthreads();
                // two 16-byte columns per thread per pass, all loads of a pass in flight together
                for (int i0 = 0; i0 < n16; i0 += 2 * kLLThreads) {
                    const int ia = i0 + tid, ib = i0 + kLLThreads + tid;
                    float acc[2][8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[0][j] = acc[1][j] = 0.f;
                    for (int k0 = 0; k0 < K; k0 += 8) {
                        int4 va[8], vb[8];
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const long long row = k < K ? s_sel_row[k] : -1;
                            const int4* base = row >= 0 ? s_base[s_sel_rank[k]] + row : nullptr;
                            va[kk] = (row >= 0 && ia < n16) ? ld_peer(base + ia) : make_int4(0, 0, 0, 0);
                            vb[kk] = (row >= 0 && ib < n16) ? ld_peer(base + ib) : make_int4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int k = k0 + kk;
                            const float w = k < K ? s_sel_w[k] : 0.f;
                            const uint32_t ua[4] = {(uint32_t)va[kk].x, (uint32_t)va[kk].y, (uint32_t)va[kk].z, (uint32_t)va[kk].w};
                            const uint32_t ub[4] = {(uint32_t)vb[kk].x, (uint32_t)vb[kk].y, (uint32_t)vb[kk].z, (uint32_t)vb[kk].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 pa = bf16x2_to_f2(ua[j]), pb = bf16x2_to_f2(ub[j]);
                                acc[0][2 * j] = fmaf(w, pa.x, acc[0][2 * j]);
                                acc[0][2 * j + 1] = fmaf(w, pa.y, acc[0][2 * j + 1]);
                                acc[1][2 * j] = fmaf(w, pb.x, acc[1][2 * j]);
                                acc[1][2 * j + 1] = fmaf(w, pb.y, acc[1][2 * j + 1]);
                            }
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int i = h == 0 ? ia : ib;
                        if (i >= n16) continue;
                        int4 o;
                        o.x = (int)f2_to_bf16x2(acc[h][0], acc[h][1]);
                        o.y = (int)f2_to_bf16x2(acc[h][2], acc[h][3]);
                        o.z = (int)f2_to_bf16x2(acc[h][4], acc[h][5]);
                        o.w = (int)f2_to_bf16x2(acc[h][6], acc[h][7]);
                        st_stream(reinterpret_cast<int4*>(a.out) + (size_t)t * n16 + i, o);
                    }
                }
            }
        }
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 5);
        // Readers of a caller-owned symmetric tensor tell its owner when they are done (the zero-copy buffer needs no such
        // hop: a rank reuses it only two dispatches later, by which time every reader has been seen to finish).
        const bool last = cta_is_last(c.local_scratch + kTicketLLCombine, gridDim.x);
        if (last) {
            if (a.close_barrier && tid < R && !s_mask[tid]) st_release_sys(&c.ctrl(tid)->barrier_in[kBarLL][me], seq);
            if (tid == 0) commit_seq(c, kFamLLCombine, seq);
        }
        if (a.close_barrier && blockIdx.x == 0 && tid < R && !s_mask[tid]) {
            if (!wait_ge_sys(&my->barrier_in[kBarLL][tid], seq, c.timeout_cycles)) report(c.status, kTimeoutBarrier, me, tid, 300);
        }
        if (traced) trace_stamp(c, kFamLLCombine, tslot, 6);
    }
    if (early) pdl_wait_predecessor();  // this kernel may not complete before its predecessor has
}

}  // namespace ll

cudaError_t launch_ll_combine(const LLCombineArgs* a, int nv, cudaStream_t stream) {
    if (a[0].pull) return DX_LAUNCH_RANKED_PDL(ll::combine_pull, LLCombineArgs, a, nv, a[0].num_sms, kLLThreads, 0, stream);
    const size_t smem = ((size_t)a[0].num_experts / a[0].ctx.num_ranks + 1) * sizeof(int);
    return DX_LAUNCH_RANKED_PDL(ll::combine, LLCombineArgs, a, nv, a[0].num_sms, kLLThreads, smem, stream);
}

}  // namespace dx
