// Expert-major dispatch for the fused MoE layer: rows land at the receiver already grouped by expert, 128-row
// aligned, in the order the grouped GEMM consumes them, and the GEMM starts on an expert as soon as its rows are in.
//
//   em_notify   every rank histograms its selections per GLOBAL expert (one warp per expert, rows of an expert keep
//               token order), all-gathers the E counts (+ the offsets of its receive buffers) with one release flag
//               per peer, and derives from the R x E matrix everything the layer needs without a host round trip:
//               where each of its (token, expert) rows goes, the group offsets of its own experts, and how many rows
//               each of its experts will receive (added to a monotonic expectation that the GEMM compares with the
//               arrival counter).
//   em_dispatch a warp takes a unit of up to 8 rows of one expert, quantises each BF16 row to e4m3 (one scale per 128
//               channels, as fp32 or as the UE8M0 words of the tensor core's scale atoms; or copies rows that were quantised
//               once per token beforehand, which is what the overlapped layer does), stores it at its final row
//               of the expert's rank, and bumps that expert's arrival counter with one release reduction. Units are
//               issued expert-major (local expert index first, then destination rank), so on every rank expert 0
//               completes first and the GEMM's group order equals the arrival order.
//   stage_reduce the home rank's sum_k w[t,k] * stage[t,k] after the second GEMM scattered its output rows into the
//               stage (grouped_gemm.cu, scatter epilogue).
// The kernels never wait on each other except for the count exchange (bounded, reports through the status word).
//
// The reference dispatches rank-major through ring queues (csrc/kernels/intranode.cu:197-610) and leaves the
// expert-major permutation to its users; it has no counterpart of the arrival gating.
#include "api.h"
#include "prims.cuh"
#include "launch.cuh"

namespace dx {

// One warp per expert scans all selections, so the scan's length is fixed; what varies is how many such warps share an SM's four
// schedulers. Four warps per CTA (64 CTAs for 256 experts) give every scanning warp a scheduler of its own.
constexpr int kEmNotifyThreads = 128;
constexpr int kEmNotifyWarps = kEmNotifyThreads / 32;
constexpr int kEmChunk = 16384;          // selections staged in shared memory per pass (uint16 expert ids)
constexpr int kTicketFused = 5;

__device__ __forceinline__ int align128(int v) { return (v + 127) & ~127; }

template <int V>
__global__ void __launch_bounds__(kEmNotifyThreads, 1) em_notify_kernel(const __grid_constant__ ArgPack<EmNotifyArgs, V> pack) {
    const EmNotifyArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk, E = a.num_experts, L = E / R;
    const int TK = T * K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t seq = next_seq(c, kFamFused);
    extern __shared__ int s_dyn[];
    uint16_t* s_sel = reinterpret_cast<uint16_t*>(s_dyn);  // [kEmChunk] expert id of a chunk of selections (0xFFFF = none)

    // ---- every CTA: one warp per expert collects that expert's selections in token order ----
    const int e = blockIdx.x * kEmNotifyWarps + warp;
    int run = 0;
    for (int c0 = 0; c0 < TK; c0 += kEmChunk) {
        const int n = min(kEmChunk, TK - c0);
        __syncthreads();
        if (((reinterpret_cast<uintptr_t>(a.topk_idx + c0)) & 15) == 0) {
            // two ids per 16-byte load
            const longlong2* src2 = reinterpret_cast<const longlong2*>(a.topk_idx + c0);
#pragma unroll 8
            for (int i = tid; i < n / 2; i += kEmNotifyThreads) {
                const longlong2 v = src2[i];
                const uint32_t lo = (v.x >= 0 && v.x < E) ? (uint32_t)v.x : 0xFFFFu, hi = (v.y >= 0 && v.y < E) ? (uint32_t)v.y : 0xFFFFu;
                reinterpret_cast<uint32_t*>(s_sel)[i] = lo | (hi << 16);
            }
            if ((n & 1) && tid == 0) {
                const int64_t v = a.topk_idx[c0 + n - 1];
                s_sel[n - 1] = (v >= 0 && v < E) ? (uint16_t)v : (uint16_t)0xFFFF;
            }
        } else {
            for (int i = tid; i < n; i += kEmNotifyThreads) {
                const int64_t v = a.topk_idx[c0 + i];
                s_sel[i] = (v >= 0 && v < E) ? (uint16_t)v : (uint16_t)0xFFFF;
            }
        }
        __syncthreads();
        if (e < E) {
            // four groups of 32 selections per step, so that four shared-memory loads and votes are in flight at a time
            for (int i0 = 0; i0 < n; i0 += 128) {
                bool hit[4];
                unsigned b[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * 32 + lane;
                    hit[u] = i < n && s_sel[i] == (uint16_t)e;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) b[u] = __ballot_sync(0xffffffffu, hit[u]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (hit[u]) {
                        const int slot = run + __popc(b[u] & ((1u << lane) - 1));
                        if (slot < T) a.sel_list[(size_t)e * T + slot] = c0 + i0 + u * 32 + lane;  // an expert is selected at most once per token
                    }
                    run += __popc(b[u]);
                }
            }
        }
    }
    if (e < E && lane == 0) a.my_counts[e] = min(run, T);

    // ---- the last CTA to finish exchanges the counts and derives the plan ----
    if (!cta_is_last(c.local_scratch + kTicketFused, gridDim.x)) return;
    int* s_cnt = s_dyn;                 // [E] my counts
    int* s_total = s_dyn + E;           // [E] rows every expert receives from all ranks
    int* s_off = s_dyn + 2 * E;         // [E] rows of ranks before me inside every expert
    int* s_base = s_dyn + 3 * E;        // [E] first row of every expert at its own rank
    __shared__ int s_ok;
    __shared__ int s_rank_rows[kMaxRanks];
    if (tid == 0) s_ok = 1;
    for (int i = tid; i < E; i += kEmNotifyThreads) s_cnt[i] = __ldcg(&a.my_counts[i]);
    __syncthreads();
    const int P = (int)(seq & 1);
    for (int d = 0; d < R; ++d) {
        ControlBlock* pc = c.ctrl(d);
        for (int i = tid; i < E; i += kEmNotifyThreads) st_relaxed_sys(&pc->em_counts[P][me][i], s_cnt[i]);
        if (tid < 4) {
            const uint64_t w = tid == 0 ? a.recv_x_off : tid == 1 ? a.recv_scales_off : tid == 2 ? a.recv_info_off : a.stage_off;
            st_relaxed_sys(&pc->em_desc[P][me][tid], w);
        }
    }
    __syncthreads();
    if (tid < R) {
        st_release_sys(&c.ctrl(tid)->em_seq[me], seq);
        if (!wait_ge_sys(&c.my_ctrl()->em_seq[tid], seq, c.timeout_cycles)) {
            report(c.status, kTimeoutFusedNotify, me, tid, 0);
            s_ok = 0;
        }
    }
    __syncthreads();
    if (s_ok) {
        ControlBlock* my = c.my_ctrl();
        for (int i = tid; i < E; i += kEmNotifyThreads) {
            int total = 0, before = 0;
            for (int src = 0; src < R; ++src) {
                const int v = ld_relaxed_sys(&my->em_counts[P][src][i]);
                total += v;
                if (src < me) before += v;
            }
            s_total[i] = total;
            s_off[i] = before;
        }
        __syncthreads();
        // first row of every expert at its rank: exclusive prefix of the 128-aligned totals, one warp per rank
        for (int d = warp; d < R; d += kEmNotifyWarps) {
            int carry = 0;
            for (int l0 = 0; l0 < L; l0 += 32) {
                const int le = l0 + lane;
                const int v = le < L ? align128(s_total[d * L + le]) : 0;
                const int incl = warp_incl_scan(v);
                if (le < L) s_base[d * L + le] = carry + incl - v;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) s_rank_rows[d] = carry;
        }
        __syncthreads();
        // Every rank computes the same row totals, so all of them see an overflow of some rank's receive buffer alike: the
        // call then moves no rows at all (no work units, empty groups, expectations unchanged) and reports the error.
        bool overflow = false;
        for (int d = 0; d < R; ++d) overflow = overflow || s_rank_rows[d] > a.rows_cap;
        if (overflow) {
            if (tid == 0) report(c.status, kBadArgument, me, -1, s_rank_rows[me]);
            for (int i = tid; i <= E; i += kEmNotifyThreads) a.unit_start[i] = 0;
            if (tid == 0) *a.unit_counter = 0;
            for (int le = tid; le <= L; le += kEmNotifyThreads) {
                a.m_offsets[le] = 0;
                if (le < L) a.m_ends[le] = 0;
            }
            __syncthreads();
            if (tid == 0) commit_seq(c, kFamFused, seq);
            return;
        }
        for (int i = tid; i < E; i += kEmNotifyThreads) a.send_base[i] = s_base[i] + s_off[i];
        for (int le = tid; le < L; le += kEmNotifyThreads) {
            const int g = me * L + le;
            a.m_offsets[le] = s_base[g];
            a.m_ends[le] = s_base[g] + s_total[g];
            // rows this expert will have received once this call's dispatch is complete (monotonic over the calls)
            c.seq[kFusedExpectedWord0 + le] += (uint64_t)s_total[g];
        }
        if (tid == 0) a.m_offsets[L] = s_rank_rows[me];
        // work units of the dispatch kernel, expert-major: order index o = local expert * R + destination rank
        if (warp == 0) {
            int carry = 0;
            for (int o0 = 0; o0 < E; o0 += 32) {
                const int o = o0 + lane;
                const int ex = o < E ? (o % R) * L + o / R : 0;
                const int v = o < E ? (s_cnt[ex] + a.unit_rows - 1) / a.unit_rows : 0;
                const int incl = warp_incl_scan(v);
                if (o < E) a.unit_start[o] = carry + incl - v;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) a.unit_start[E] = carry;
        }
        if (tid == 0) *a.unit_counter = 0;
        if (tid < 4 * R) {
            const int which = tid / R, r = tid % R;
            a.peer_bases[tid] = reinterpret_cast<uint64_t>(c.at<char>(r, ld_relaxed_sys(&my->em_desc[P][r][which])));
        }
    }
    if (tid == 0) commit_seq(c, kFamFused, seq);
}

cudaError_t launch_em_notify(const EmNotifyArgs* a, int nv, cudaStream_t stream) {
    const int E = a[0].num_experts;
    if (E < 1 || E > kMaxFusedExperts || E % a[0].ctx.num_ranks != 0 || a[0].unit_rows < 1) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(kEmChunk * 2 > 4 * E * 4 ? kEmChunk * 2 : 4 * E * 4);
    const int ctas = (E + kEmNotifyWarps - 1) / kEmNotifyWarps;
    return DX_LAUNCH_RANKED(em_notify_kernel, EmNotifyArgs, a, nv, ctas, kEmNotifyThreads, smem, stream);
}

// =============================================================================================
// dispatch
// =============================================================================================
constexpr int kEmDispatchThreads = 128;  // small CTAs with few registers: they share SMs with the persistent GEMM CTAs
constexpr int kEmDispatchWarps = kEmDispatchThreads / 32;

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int V>
__global__ void __launch_bounds__(kEmDispatchThreads, 6) em_dispatch_kernel(const __grid_constant__ ArgPack<EmDispatchArgs, V> pack) {
    const EmDispatchArgs& a = pack.a[blockIdx.y];
    const RankCtx& c = a.ctx;
    const int R = c.num_ranks, me = c.rank, T = a.num_tokens, K = a.num_topk, E = a.num_experts, L = E / R, H = a.hidden;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    extern __shared__ int s_unit_start[];  // [E+1]
    for (int i = tid; i <= E; i += kEmDispatchThreads) s_unit_start[i] = a.unit_start[i];
    __syncthreads();
    if (a.trace != nullptr && tid == 0) atomicMin(&a.trace[0], global_timer());
    const int total_units = s_unit_start[E];
    const int num_kb = H / 128;
    char* const* rows_base = reinterpret_cast<char* const*>(a.peer_bases);
    char* const* scales_base = reinterpret_cast<char* const*>(a.peer_bases + R);
    int* const* info_base = reinterpret_cast<int* const*>(a.peer_bases + 2 * R);

    // Units are handed out through one counter (reset by the count exchange), so they are taken in order by whichever warps
    // are running: experts complete in order even when only part of the grid is resident next to a GEMM.
    while (true) {
        int u = 0;
        if (lane == 0) u = atomicAdd(a.unit_counter, 1);
        u = __shfl_sync(0xffffffffu, u, 0);
        if (u >= total_units) break;
        int lo = 0, hi = E;  // largest o with unit_start[o] <= u
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_unit_start[mid] <= u) lo = mid;
            else hi = mid;
        }
        const int o = lo, d = o % R, le = o / R, e = d * L + le;
        const int s0 = (u - s_unit_start[o]) * a.unit_rows;
        const int cnt = a.my_counts[e];
        const int n = min(a.unit_rows, cnt - s0);
        const int base_row = a.send_base[e] + s0;
        char* dst_rows = rows_base[d];
        char* dst_scales = scales_base[d];
        int sent = 0;
        for (int s = 0; s < n; ++s) {
            const int sel = a.sel_list[(size_t)e * T + s0 + s];
            const int t = sel / K;
            const int row = base_row + s;
            if (c.debug_extent != 0 && !peer_range_ok(c, d, dst_rows + (size_t)row * H, (size_t)H, 6)) continue;
            char* drow = dst_rows + (size_t)row * H;
            if (a.x_scales != nullptr) {
                // rows quantised beforehand (once per token instead of once per selection): a pure copy, 4 KiB per pass
                const int n16 = H / 16;
                const int4* src16 = reinterpret_cast<const int4*>(reinterpret_cast<const char*>(a.x) + (size_t)t * H);
                for (int i0 = 0; i0 < n16; i0 += 256) {
                    int4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int i = i0 + u * 32 + lane;
                        if (i < n16) v[u] = ld_cached(src16 + i);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int i = i0 + u * 32 + lane;
                        if (i < n16) st_stream(reinterpret_cast<int4*>(drow) + i, v[u]);
                    }
                }
                for (int kb = lane; kb < num_kb; kb += 32) {
                    const float scale = a.x_scales[(size_t)t * num_kb + kb];
                    if (a.native_atoms) {
                        const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
                        *reinterpret_cast<uint32_t*>(dst_scales + ((size_t)(row >> 7) * num_kb + kb) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4) =
                            ex * 0x01010101u;
                    } else {
                        reinterpret_cast<float*>(dst_scales)[(size_t)row * num_kb + kb] = scale;
                    }
                }
                if (lane == 0) {
                    info_base[d][row] = (me << 24) | sel;
                    if (a.dst_row != nullptr) a.dst_row[sel] = row;
                }
                ++sent;
                continue;
            }
            const char* src = reinterpret_cast<const char*>(a.x) + (size_t)t * H * 2;
            // a lane owns 16 consecutive channels, 8 lanes share a scale, a warp covers 512 channels per half step; the loads
            // of the next 1024 channels are issued before the current ones are converted
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
                    const int4 q0 = cur[2 * h], q1 = cur[2 * h + 1];
                    const uint32_t w[8] = {(uint32_t)q0.x, (uint32_t)q0.y, (uint32_t)q0.z, (uint32_t)q0.w,
                                           (uint32_t)q1.x, (uint32_t)q1.y, (uint32_t)q1.z, (uint32_t)q1.w};
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
                    fp8_scale_from_amax(amax, a.round_scale != 0 || a.native_atoms != 0, scale, inv);
                    int4 q;
                    q.x = (int)pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                    q.y = (int)pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                    q.z = (int)pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
                    q.w = (int)pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
                    if (act) {
                        st_stream(reinterpret_cast<int4*>(drow + ch), q);
                        if ((lane & 7) == 0) {
                            const int kb = ch >> 7;
                            if (a.native_atoms) {
                                // UE8M0 word of the scale atom of (128-row tile, K block): row m0 + 32*m1 sits at m0*16 + m1*4
                                const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
                                *reinterpret_cast<uint32_t*>(dst_scales + ((size_t)(row >> 7) * num_kb + kb) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4) =
                                    ex * 0x01010101u;
                            } else {
                                reinterpret_cast<float*>(dst_scales)[(size_t)row * num_kb + kb] = scale;
                            }
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
            }
            if (lane == 0) {
                info_base[d][row] = (me << 24) | sel;
                if (a.dst_row != nullptr) a.dst_row[sel] = row;
            }
            ++sent;
        }
        __syncwarp();
        // one release per unit: everything this warp stored for expert (d, le) is visible before the counter moves
        if (lane == 0 && sent > 0) red_add_release_sys(&c.ctrl(d)->em_arrived[le], (uint64_t)sent);
    }
    if (a.trace != nullptr) {
        __syncthreads();
        if (tid == 0) atomicMax(&a.trace[1], global_timer());
    }
}

cudaError_t launch_em_dispatch(const EmDispatchArgs* a, int nv, cudaStream_t stream) {
    if (a[0].hidden % 128 != 0 || a[0].num_sms < 1) return cudaErrorInvalidValue;
    const size_t smem = (size_t)(a[0].num_experts + 1) * sizeof(int);
    return DX_LAUNCH_RANKED(em_dispatch_kernel, EmDispatchArgs, a, nv, a[0].num_sms, kEmDispatchThreads, smem, stream);
}

// =============================================================================================
// home-side reduction of the scattered expert outputs
// =============================================================================================
constexpr int kStageReduceThreads = 256;

// out[t] = sum_k w[t,k] * stage[t*K + k] over the valid selections of token t (fp32 accumulate, fixed k order).
__global__ void __launch_bounds__(kStageReduceThreads) stage_reduce_kernel(const __nv_bfloat16* __restrict__ stage, __nv_bfloat16* __restrict__ out,
                                                                          const int64_t* __restrict__ topk_idx, const float* __restrict__ w,
                                                                          int num_tokens, int num_topk, int num_experts, int hidden) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (kStageReduceThreads / 32) + (threadIdx.x >> 5);
    if (t >= num_tokens) return;
    const int n16 = hidden / 8;
    bool ok = false;
    float my_w = 0.f;
    if (lane < num_topk) {
        const int64_t e = topk_idx[(size_t)t * num_topk + lane];
        ok = e >= 0 && e < num_experts;
        my_w = ok ? w[(size_t)t * num_topk + lane] : 0.f;
    }
    const unsigned valid = __ballot_sync(0xffffffffu, ok);
    const int4* rows = reinterpret_cast<const int4*>(stage) + (size_t)t * num_topk * n16;
    int4* d = reinterpret_cast<int4*>(out) + (size_t)t * n16;
    constexpr int U = 2;
    for (int i0 = 0; i0 < n16; i0 += 32 * U) {
        float acc[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
        // eight selections x two columns: sixteen 16-byte loads in flight per lane before the first one is consumed
        for (int k0 = 0; k0 < num_topk; k0 += 8) {
            int4 v[8][U];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const int k = k0 + kk;
                const bool kv = k < num_topk && ((valid >> k) & 1u);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + u * 32 + lane;
                    v[kk][u] = (kv && i < n16) ? ld_stream(rows + (size_t)k * n16 + i) : make_int4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const float wk = __shfl_sync(0xffffffffu, my_w, (k0 + kk) & 31);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t w4[4] = {(uint32_t)v[kk][u].x, (uint32_t)v[kk][u].y, (uint32_t)v[kk][u].z, (uint32_t)v[kk][u].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = bf16x2_to_f2(w4[q]);
                        acc[u][2 * q] = fmaf(wk, f.x, acc[u][2 * q]);
                        acc[u][2 * q + 1] = fmaf(wk, f.y, acc[u][2 * q + 1]);
                    }
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

cudaError_t launch_stage_reduce(const void* stage, void* out, const int64_t* topk_idx, const float* w, int num_tokens, int num_topk,
                                int num_experts, int hidden, cudaStream_t stream) {
    if (num_tokens <= 0) return cudaSuccess;
    if (hidden % 8 != 0 || num_topk < 1 || num_topk > 32) return cudaErrorInvalidValue;
    const int per = kStageReduceThreads / 32;
    stage_reduce_kernel<<<(num_tokens + per - 1) / per, kStageReduceThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(stage), static_cast<__nv_bfloat16*>(out), topk_idx, w, num_tokens, num_topk, num_experts, hidden);
    return cudaGetLastError();
}

}  // namespace dx
