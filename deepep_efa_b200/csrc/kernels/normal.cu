// Normal (high-throughput) mode over one NVSwitch domain: notify, dispatch, combine, barrier.
//
// Design (differs from the reference on purpose):
//  * No ring queues, no channels, no flow control. With 180 GB per GPU the receiver's FINAL output
//    tensors live in its peer-mapped symmetric arena, and a count exchange tells every sender the
//    exact destination row of every token before any payload moves. Senders then store rows straight
//    into the peers' final tensors (push, 16-byte stores, optional fused BF16->FP8 block quantisation)
//    and the receiver never touches the payload.
//  * Combine is the mirror image as a PULL: the token's home rank loads the <= R expert-output rows
//    from the peers' symmetric memory, reduces them in fp32 (+bias), and writes BF16 once.
//  * Completion is one cross-rank sequence barrier at the end of each kernel; all sequence numbers
//    are monotonic, so nothing is cleaned between calls.
//  * Every wait is bounded and reports through the status word.
//
// Row order at the receiver is (source rank, source token order), which is exactly the order the
// reference produces with its (rank, channel, token) rings because channels are contiguous token
// ranges (csrc/kernels/intranode.cu:410-426, 464).
//
// Reference counterparts: notify_dispatch / cached_notify_dispatch (intranode.cu:11-195),
// dispatch (:197-610), cached_notify_combine / combine (:612-1099), intranode::barrier (runtime.cu:13-26).
#include "api.h"
#include "prims.cuh"
#include "launch.cuh"

namespace dx {

// Indices into RankCtx::local_scratch (ints, zero between kernels).
constexpr int kTicketDispatch = 0;
constexpr int kTicketCombine = 1;
constexpr int kTicketNotify = 2;

// =============================================================================================
// notify
// =============================================================================================
constexpr int kNotifyThreads = 1024;

template <int V>
__global__ void __launch_bounds__(kNotifyThreads, 1) notify_kernel(const __grid_constant__ ArgPack<NotifyArgs, V> pack) {
    const NotifyArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank;
    const int E = a.num_experts, L = E / R, C = a.num_channels, T = a.num_tokens;
    const int tid = threadIdx.x;
    const uint64_t seq = next_seq(c, kFamNotify);
    __shared__ int s_ok;
    __shared__ int s_warp_sums[kNotifyThreads / 32];
    __shared__ int s_off[kNotifyThreads + 1];

    if (blockIdx.x == 0) {
        // ---- CTA 0: exchange counts with every rank, build the prefix matrix, tell the host ----
        if (tid == 0) s_ok = 1;
        for (int d = 0; d < R; ++d) {
            ControlBlock* pc = c.ctrl(d);
            if (tid < R) st_relaxed_sys(&pc->notify_rank_counts[me][tid], a.num_tokens_per_rank[tid]);
            for (int i = tid; i < L; i += kNotifyThreads)
                st_relaxed_sys(&pc->notify_expert_counts[me][i], a.num_tokens_per_expert[d * L + i]);
        }
        __syncthreads();
        if (tid < R) {
            st_release_sys(&c.ctrl(tid)->notify_seq[me], seq);
            if (!wait_ge_sys(&c.my_ctrl()->notify_seq[tid], seq, c.timeout_cycles)) {
                report(c.status, kTimeoutNotify, me, tid, 0);
                s_ok = 0;
            }
        }
        __syncthreads();
        if (!s_ok) {
            if (tid == 0) {
                *a.host_recv_counter = -2;  // tells the host to stop waiting
                __threadfence_system();
            }
            return;
        }
        ControlBlock* my = c.my_ctrl();
        if (tid < R) {
            int running = 0;
            for (int i = 0; i < R; ++i) {
                running += ld_relaxed_sys(&my->notify_rank_counts[i][tid]);
                a.rank_prefix_matrix[i * R + tid] = running;
            }
            if (tid == me) *a.host_recv_counter = running;
        }
        for (int e = tid; e < L; e += kNotifyThreads) {
            int sum = 0;
            for (int i = 0; i < R; ++i) sum += ld_relaxed_sys(&my->notify_expert_counts[i][e]);
            const int al = a.expert_alignment;
            a.host_expert_counter[e] = (sum + al - 1) / al * al;
        }
        __threadfence_system();
        // channel prefix rows pushed by the scan CTAs of my peers
        if (tid < R) {
            uint64_t dummy;
            if (!mailbox_wait(c, kMbChanPrefix, tid, seq, &dummy, 0)) {
                report(c.status, kTimeoutNotify, me, tid, 1);
                s_ok = 0;
            }
        }
        __syncthreads();
        if (!s_ok) return;
        for (int i = tid; i < R * C; i += kNotifyThreads)
            a.recv_channel_prefix_matrix[i] = ld_relaxed_sys(&my->chan_prefix_in[i / C][i % C]);
        if (cta_is_last(c.local_scratch + kTicketNotify, gridDim.x) && tid == 0) commit_seq(c, kFamNotify, seq);
        return;
    }

    // ---- CTA 1+d: positions of my tokens inside the (me -> d) stream ----
    const int d = blockIdx.x - 1;
    const int per = (T + kNotifyThreads - 1) / kNotifyThreads;
    const int begin = min(tid * per, T), end = min(begin + per, T);
    int cnt = 0;
    for (int t = begin; t < end; ++t) cnt += a.is_token_in_rank[(size_t)t * R + d] ? 1 : 0;
    // block exclusive scan of cnt
    const int incl = warp_incl_scan(cnt);
    if ((tid & 31) == 31) s_warp_sums[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        const int w = s_warp_sums[tid];
        const int wi = warp_incl_scan(w);
        s_warp_sums[tid] = wi - w;
    }
    __syncthreads();
    int pos = s_warp_sums[tid >> 5] + incl - cnt;
    // keep exclusive offsets for the channel prefix computation
    s_off[tid] = pos;
    if (tid == kNotifyThreads - 1) s_off[kNotifyThreads] = pos + cnt;
    for (int t = begin; t < end; ++t) {
        const bool in = a.is_token_in_rank[(size_t)t * R + d];
        a.send_head[(size_t)t * R + d] = in ? pos : -1;
        pos += in ? 1 : 0;
    }
    __syncthreads();
    // channel ch covers tokens [ch*tpc, min((ch+1)*tpc, T)); prefix = tokens to d in channels <= ch
    const int tpc = (T + C - 1) / C;
    if (tid < C) {
        const int b = min((tid + 1) * tpc, T);  // count flagged tokens with index < b
        int owner = per > 0 ? b / per : 0;
        if (owner > kNotifyThreads) owner = kNotifyThreads;
        int prefix = s_off[owner];
        if (owner < kNotifyThreads)
            for (int t = owner * per; t < b; ++t) prefix += a.is_token_in_rank[(size_t)t * R + d] ? 1 : 0;
        a.channel_prefix_matrix[d * C + tid] = prefix;
        st_relaxed_sys(&c.ctrl(d)->chan_prefix_in[me][tid], prefix);
    }
    __syncthreads();
    if (tid == 0) {
        mailbox_post(c, kMbChanPrefix, d, nullptr, 0, seq);
    }
    if (cta_is_last(c.local_scratch + kTicketNotify, gridDim.x) && tid == 0) commit_seq(c, kFamNotify, seq);
}

cudaError_t launch_notify(const NotifyArgs* a, int nv, cudaStream_t stream) {
    return DX_LAUNCH_RANKED(notify_kernel, NotifyArgs, a, nv, 1 + a[0].ctx.num_ranks, kNotifyThreads, 0, stream);
}

// =============================================================================================
// dispatch (push)
// =============================================================================================
constexpr int kDispatchThreads = 1024;
constexpr int kDispatchWarps = kDispatchThreads / 32;

struct PeerDst {
    char* x;
    float* scales;
    int64_t* topk_idx;
    float* topk_w;
    int* src_idx;
    int base_row;  // rows of ranks before me at that peer
};

template <int V>
__global__ void __launch_bounds__(kDispatchThreads, 1) dispatch_kernel(const __grid_constant__ ArgPack<DispatchArgs, V> pack) {
    const DispatchArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk;
    const int L = a.num_experts / R;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t seq = next_seq(c, kFamDispatch);
    __shared__ PeerDst s_dst[kMaxRanks];
    __shared__ int s_ok;
    __shared__ float s_scales[kDispatchWarps][64];

    if (tid == 0) s_ok = 1;
    __syncthreads();
    // Publish where my rows go, then learn where every peer wants its rows.
    if (blockIdx.x == 0 && tid < R) {
        uint64_t w[5] = {a.recv_x_off, a.recv_scales_off, a.recv_topk_idx_off, a.recv_topk_w_off, a.recv_src_idx_off};
        mailbox_post(c, kMbDispatchDesc, tid, w, 5, seq);
    }
    if (tid < R) {
        uint64_t w[5];
        if (!mailbox_wait(c, kMbDispatchDesc, tid, seq, w, 5)) {
            report(c.status, kTimeoutDescriptor, me, tid, 0);
            s_ok = 0;
        } else {
            PeerDst p;
            p.x = c.at<char>(tid, w[0]);
            p.scales = c.at<float>(tid, w[1]);
            p.topk_idx = c.at<int64_t>(tid, w[2]);
            p.topk_w = c.at<float>(tid, w[3]);
            p.src_idx = c.at<int>(tid, w[4]);
            p.base_row = me > 0 ? a.rank_prefix_matrix[(me - 1) * R + tid] : 0;
            s_dst[tid] = p;
        }
    }
    __syncthreads();
    if (!s_ok) return;

    const int H = a.hidden;
    const bool quant = a.quantize != 0;
    const int out_elem = quant ? 1 : a.x_elem_bytes;
    const size_t out_row_bytes = (size_t)H * out_elem;
    const int num_scales = H / 128;
    const bool has_scales = quant || a.x_scales != nullptr;
    const int total_warps = a.num_sms * kDispatchWarps;

    for (int t = blockIdx.x * kDispatchWarps + warp; t < T; t += total_warps) {
        // destination rows
        int head = (lane < R) ? a.send_head[(size_t)t * R + lane] : -1;
        const unsigned dmask = __ballot_sync(0xffffffffu, head >= 0);
        if (dmask == 0) continue;
        int rows[kMaxRanks];
#pragma unroll
        for (int d = 0; d < kMaxRanks; ++d) {
            const int h = __shfl_sync(0xffffffffu, head, d);
            rows[d] = (d < R && h >= 0) ? s_dst[d].base_row + h : -1;
            if (c.debug_extent != 0 && rows[d] >= 0 &&
                !peer_range_ok(c, d, s_dst[d].x + (size_t)rows[d] * ((size_t)a.hidden * (a.quantize != 0 ? 1 : a.x_elem_bytes)),
                               (size_t)a.hidden * (a.quantize != 0 ? 1 : a.x_elem_bytes), 1))
                rows[d] = -1;
        }

        if (!quant) {
            // ---- pass-through rows (bf16 or already-quantised e4m3) ----
            const int n16 = (int)(out_row_bytes / 16);
            const int4* src = reinterpret_cast<const int4*>(reinterpret_cast<const char*>(a.x) + (size_t)t * out_row_bytes);
            constexpr int U = 4;
            for (int i0 = 0; i0 < n16; i0 += 32 * U) {
                int4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    if (i < n16) v[u] = ld_stream(src + i);
                }
#pragma unroll
                for (int d = 0; d < kMaxRanks; ++d) {
                    if (rows[d] < 0) continue;
                    int4* dst = reinterpret_cast<int4*>(s_dst[d].x + (size_t)rows[d] * out_row_bytes);
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int i = i0 + u * 32 + lane;
                        if (i < n16) st_stream(dst + i, v[u]);
                    }
                }
            }
            if (a.x_scales != nullptr) {
                for (int i = lane; i < num_scales; i += 32) {
                    const float s = a.x_scales[(size_t)t * num_scales + i];
#pragma unroll
                    for (int d = 0; d < kMaxRanks; ++d)
                        if (rows[d] >= 0) s_dst[d].scales[(size_t)rows[d] * num_scales + i] = s;
                }
            }
        } else {
            // ---- fused BF16 -> e4m3 with one fp32 scale per 128 channels ----
            // A lane owns 16 consecutive channels, 8 lanes own one scale group, a warp covers 512
            // channels per step.
            const char* src = reinterpret_cast<const char*>(a.x) + (size_t)t * H * 2;
            // four 16-byte loads per lane in flight: the next 1024 channels are requested before the current ones are converted
            int4 cur[4], nxt[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int ch = h * 512 + lane * 16;
                cur[2 * h] = cur[2 * h + 1] = make_int4(0, 0, 0, 0);
                if (ch < H) {
                    cur[2 * h] = ld_cached(reinterpret_cast<const int4*>(src + (size_t)ch * 2));
                    cur[2 * h + 1] = ld_cached(reinterpret_cast<const int4*>(src + (size_t)ch * 2 + 16));
                }
            }
            for (int c0 = 0; c0 < H; c0 += 1024) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int chn = c0 + 1024 + h * 512 + lane * 16;
                    nxt[2 * h] = nxt[2 * h + 1] = make_int4(0, 0, 0, 0);
                    if (chn < H) {
                        nxt[2 * h] = ld_cached(reinterpret_cast<const int4*>(src + (size_t)chn * 2));
                        nxt[2 * h + 1] = ld_cached(reinterpret_cast<const int4*>(src + (size_t)chn * 2 + 16));
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int ch = c0 + h * 512 + lane * 16;
                    const bool act = ch < H;
                    const int4 r0 = cur[2 * h], r1 = cur[2 * h + 1];
                    float f[16];
                    {
                        const uint32_t w[8] = {(uint32_t)r0.x, (uint32_t)r0.y, (uint32_t)r0.z, (uint32_t)r0.w,
                                               (uint32_t)r1.x, (uint32_t)r1.y, (uint32_t)r1.z, (uint32_t)r1.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float2 p = bf16x2_to_f2(w[j]);
                            f[2 * j] = p.x;
                            f[2 * j + 1] = p.y;
                        }
                    }
                    float amax = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    float scale, inv;
                    fp8_scale_from_amax(amax, a.round_scale != 0, scale, inv);
                    int4 q;
                    q.x = (int)pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                    q.y = (int)pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                    q.z = (int)pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                    q.w = (int)pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                    if (act && (lane & 7) == 0) s_scales[warp][ch >> 7] = scale;
                    if (act) {
#pragma unroll
                        for (int d = 0; d < kMaxRanks; ++d)
                            if (rows[d] >= 0) st_stream(reinterpret_cast<int4*>(s_dst[d].x + (size_t)rows[d] * H + ch), q);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
            }
            __syncwarp();
            for (int i = lane; i < num_scales; i += 32) {
                const float s = s_scales[warp][i];
#pragma unroll
                for (int d = 0; d < kMaxRanks; ++d)
                    if (rows[d] >= 0) s_dst[d].scales[(size_t)rows[d] * num_scales + i] = s;
            }
            __syncwarp();
        }
        (void)has_scales;

        // ---- metadata: local expert ids, weights, source token index ----
        if (a.topk_idx != nullptr && lane < K) {
            const int64_t e = a.topk_idx[(size_t)t * K + lane];
            const float w = a.topk_weights != nullptr ? a.topk_weights[(size_t)t * K + lane] : 0.f;
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d) {
                if (rows[d] < 0) continue;
                const bool mine = e >= (int64_t)d * L && e < (int64_t)(d + 1) * L;
                s_dst[d].topk_idx[(size_t)rows[d] * K + lane] = mine ? e - (int64_t)d * L : -1;
                if (a.topk_weights != nullptr) s_dst[d].topk_w[(size_t)rows[d] * K + lane] = mine ? w : 0.f;
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d)
                if (rows[d] >= 0) s_dst[d].src_idx[rows[d]] = t;
        }
    }

    // worst-case sized outputs: mark the unused tail of my own recv_topk_idx
    if (a.num_worst_tokens > 0 && a.topk_idx != nullptr) {
        const int num_recv = a.rank_prefix_matrix[(R - 1) * R + me];
        int64_t* mine = c.at<int64_t>(me, a.recv_topk_idx_off);
        const size_t lo = (size_t)num_recv * K, hi = (size_t)a.num_worst_tokens * K;
        for (size_t i = lo + (size_t)blockIdx.x * kDispatchThreads + tid; i < hi; i += (size_t)a.num_sms * kDispatchThreads)
            mine[i] = -1;
    }

    // ---- completion: when my last CTA is done, tell every peer; CTA 0 waits for every peer ----
    if (cta_is_last(c.local_scratch + kTicketDispatch, gridDim.x)) {
        if (tid < R) {
            st_release_sys(&c.ctrl(tid)->barrier_in[kBarDispatch][me], seq);
        }
        if (tid == 0) commit_seq(c, kFamDispatch, seq);
    }
    if (blockIdx.x == 0 && tid < R) {
        if (!wait_ge_sys(&c.my_ctrl()->barrier_in[kBarDispatch][tid], seq, c.timeout_cycles))
            report(c.status, kTimeoutBarrier, me, tid, 100);
    }
}

cudaError_t launch_dispatch(const DispatchArgs* a, int nv, cudaStream_t stream) {
    return DX_LAUNCH_RANKED(dispatch_kernel, DispatchArgs, a, nv, a[0].num_sms, kDispatchThreads, 0, stream);
}

// =============================================================================================
// combine (pull)
// =============================================================================================
constexpr int kCombineThreads = 512;
constexpr int kCombineWarps = kCombineThreads / 32;

struct PeerSrc {
    const int4* x;
    const float* w;
    int base_row;
};

template <int kRanks>
__device__ __forceinline__ void combine_rows(const CombineArgs& a, const PeerSrc* s_src, int warp, int lane, int R) {
    const int T = a.num_tokens, H = a.hidden, K = a.num_topk;
    const int n16 = H / 8;
    const int total_warps = a.num_sms * kCombineWarps;
    constexpr int U = 2;
    for (int t = blockIdx.x * kCombineWarps + warp; t < T; t += total_warps) {
        int head = (lane < R) ? a.send_head[(size_t)t * R + lane] : -1;
        const int4* rowp[kRanks];
        const float* wp[kRanks];
#pragma unroll
        for (int r = 0; r < kRanks; ++r) {
            const int h = __shfl_sync(0xffffffffu, head, r);
            const bool ok = r < R && h >= 0;
            rowp[r] = ok ? s_src[r].x + (size_t)(s_src[r].base_row + h) * n16 : nullptr;
            if (a.ctx.debug_extent != 0 && ok && !peer_range_ok(a.ctx, r, rowp[r], (size_t)n16 * 16, 2)) rowp[r] = nullptr;
            wp[r] = (ok && rowp[r] != nullptr && s_src[r].w != nullptr) ? s_src[r].w + (size_t)(s_src[r].base_row + h) * K : nullptr;
        }
        const int4* b0 = a.bias0 ? reinterpret_cast<const int4*>(a.bias0) + (size_t)t * n16 : nullptr;
        const int4* b1 = a.bias1 ? reinterpret_cast<const int4*>(a.bias1) + (size_t)t * n16 : nullptr;
        int4* out = reinterpret_cast<int4*>(a.out) + (size_t)t * n16;
        for (int i0 = 0; i0 < n16; i0 += 32 * U) {
            int4 v[kRanks][U];
#pragma unroll
            for (int r = 0; r < kRanks; ++r) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    v[r][u] = (rowp[r] != nullptr && i < n16) ? ld_peer(rowp[r] + i) : make_int4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32 + lane;
                if (i >= n16) continue;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int r = 0; r < kRanks; ++r) {
                    const uint32_t w[4] = {(uint32_t)v[r][u].x, (uint32_t)v[r][u].y, (uint32_t)v[r][u].z, (uint32_t)v[r][u].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 p = bf16x2_to_f2(w[j]);
                        acc[2 * j] += p.x;
                        acc[2 * j + 1] += p.y;
                    }
                }
                if (b0 != nullptr) {
                    const int4 b = ld_cached(b0 + i);
                    const uint32_t w[4] = {(uint32_t)b.x, (uint32_t)b.y, (uint32_t)b.z, (uint32_t)b.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 p = bf16x2_to_f2(w[j]);
                        acc[2 * j] += p.x;
                        acc[2 * j + 1] += p.y;
                    }
                }
                if (b1 != nullptr) {
                    const int4 b = ld_cached(b1 + i);
                    const uint32_t w[4] = {(uint32_t)b.x, (uint32_t)b.y, (uint32_t)b.z, (uint32_t)b.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 p = bf16x2_to_f2(w[j]);
                        acc[2 * j] += p.x;
                        acc[2 * j + 1] += p.y;
                    }
                }
                int4 o;
                o.x = (int)f2_to_bf16x2(acc[0], acc[1]);
                o.y = (int)f2_to_bf16x2(acc[2], acc[3]);
                o.z = (int)f2_to_bf16x2(acc[4], acc[5]);
                o.w = (int)f2_to_bf16x2(acc[6], acc[7]);
                st_stream(out + i, o);
            }
        }
        if (a.out_topk_w != nullptr && lane < K) {
            float sum = 0.f;
#pragma unroll
            for (int r = 0; r < kRanks; ++r)
                if (wp[r] != nullptr) sum += __int_as_float(ld_relaxed_sys(reinterpret_cast<const int*>(wp[r] + lane)));
            a.out_topk_w[(size_t)t * K + lane] = sum;
        }
    }
}

template <int V>
__global__ void __launch_bounds__(kCombineThreads, 1) combine_kernel(const __grid_constant__ ArgPack<CombineArgs, V> pack) {
    const CombineArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t seq = next_seq(c, kFamCombine);
    __shared__ PeerSrc s_src[kMaxRanks];
    __shared__ int s_ok;
    if (tid == 0) s_ok = 1;
    __syncthreads();
    // "my expert outputs are final and live at this offset" -> every home rank
    if (blockIdx.x == 0 && tid < R) {
        uint64_t w[2] = {a.x_off, a.topk_w_off};
        mailbox_post(c, kMbCombineSrc, tid, w, 2, seq);
    }
    if (tid < R) {
        uint64_t w[2];
        if (!mailbox_wait(c, kMbCombineSrc, tid, seq, w, 2)) {
            report(c.status, kTimeoutCombineReady, me, tid, 0);
            s_ok = 0;
        } else {
            PeerSrc p;
            p.x = c.at<const int4>(tid, w[0]);
            p.w = (w[1] == ~0ull) ? nullptr : c.at<const float>(tid, w[1]);
            p.base_row = me > 0 ? a.rank_prefix_matrix[(me - 1) * R + tid] : 0;
            s_src[tid] = p;
        }
    }
    __syncthreads();
    if (!s_ok) return;

    if (R <= 1) combine_rows<1>(a, s_src, warp, lane, R);
    else if (R <= 2) combine_rows<2>(a, s_src, warp, lane, R);
    else if (R <= 4) combine_rows<4>(a, s_src, warp, lane, R);
    else combine_rows<8>(a, s_src, warp, lane, R);

    // Peers may reuse their expert-output buffers only after every home rank has finished reading.
    if (cta_is_last(c.local_scratch + kTicketCombine, gridDim.x)) {
        if (tid < R) {
            st_release_sys(&c.ctrl(tid)->barrier_in[kBarCombine][me], seq);
        }
        if (tid == 0) commit_seq(c, kFamCombine, seq);
    }
    if (blockIdx.x == 0 && tid < R) {
        if (!wait_ge_sys(&c.my_ctrl()->barrier_in[kBarCombine][tid], seq, c.timeout_cycles))
            report(c.status, kTimeoutBarrier, me, tid, 200);
    }
}

cudaError_t launch_combine(const CombineArgs* a, int nv, cudaStream_t stream) {
    return DX_LAUNCH_RANKED(combine_kernel, CombineArgs, a, nv, a[0].num_sms, kCombineThreads, 0, stream);
}

// =============================================================================================
// barrier / timeout probe
// =============================================================================================
template <int V>
__global__ void __launch_bounds__(32, 1) barrier_kernel(const __grid_constant__ ArgPack<BarrierArgs, V> pack) {
    const BarrierArgs& a = pack.a[blockIdx.y];
    const uint64_t seq = next_seq(a.ctx, kFamBarrier);
    cta_rank_barrier(a.ctx, seq);
    if (threadIdx.x == 0) commit_seq(a.ctx, kFamBarrier, seq);
}

cudaError_t launch_barrier(const BarrierArgs* a, int nv, cudaStream_t stream) {
    return DX_LAUNCH_RANKED(barrier_kernel, BarrierArgs, a, nv, 1, 32, 0, stream);
}

__global__ void timeout_probe_kernel(const RankCtx c, uint64_t* flag) {
    if (!wait_ge_sys(flag, 1, c.timeout_cycles)) report(c.status, kTimeoutTest, c.rank, -1, 0);
}

cudaError_t launch_timeout_probe(const RankCtx& ctx, uint64_t* never_set_flag, cudaStream_t stream) {
    timeout_probe_kernel<<<1, 1, 0, stream>>>(ctx, never_set_flag);
    return cudaGetLastError();
}

}  // namespace dx
