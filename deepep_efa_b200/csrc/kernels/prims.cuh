// Device-side primitives shared by every kernel of this library (sm_100a only).
//
// Everything that crosses a GPU boundary goes through the helpers in this file:
//  * payload moves as plain 16-byte global stores/loads on peer-mapped memory (never TMA),
//  * publication is a system-scope release store or release reduction on a word that lives in the
//    CONSUMER's memory, and the consumer polls its own memory with system-scope acquire loads,
//  * every poll is bounded: when the limit runs out the waiter records an error code and returns,
//    it never traps and never spins forever.
//
// The reference keeps the equivalent helpers in csrc/kernels/utils.cuh (ld/st wrappers :80-297,
// barrier_block :504-534, FP8 scale math :467-502) and csrc/transport/gdr_flags.cuh; those trap on
// timeout (utils.cuh:528-531), this file reports a status instead.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "types.h"

namespace dx {

// ---------------------------------------------------------------------------------------------
// system-scope memory operations
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_add_release_sys(uint64_t* p, uint64_t v) {
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_gpu(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// 16-byte payload moves. Loads of read-once local data skip L1 allocation; stores to peers are plain
// weak stores (ordering comes from the release that follows them).
__device__ __forceinline__ int4 ld_stream(const int4* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ int4 ld_cached(const int4* p) { return __ldg(p); }
// Peer data that another GPU wrote during this kernel: must not hit a stale L1 line and must not use
// the non-coherent path.
__device__ __forceinline__ int4 ld_peer(const int4* p) {
    int4 v;
    asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_stream(int4* p, const int4& v) {
    asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// bounded waiting
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void report(StatusBlock* sb, int code, int rank, int peer, int detail) {
    if (sb == nullptr) return;
    // Plain stores to mapped host memory (no PCIe atomics needed); an earlier error is kept.
    volatile StatusBlock* v = sb;
    if (v->code == 0) {
        v->rank = rank;
        v->peer = peer;
        v->detail = detail;
        v->code = code;
        __threadfence_system();
    }
}

// Spins on `*flag >= want` (acquire, system scope) for at most `limit` clock cycles.
// Returns true when the value arrived.
// Debug aid (RankCtx::debug_extent != 0, env DEEPEP_DEBUG_CHECKS=1): is [p, p+bytes) inside rank r's symmetric buffer?
// A violation is reported through the status block and the caller skips the access, so a corrupted handle or a wrong
// size shows up as an error code on the host instead of as a fault on a peer's GPU.
__device__ __forceinline__ bool peer_range_ok(const RankCtx& c, int r, const void* p, size_t bytes, int detail) {
    if (c.debug_extent == 0) return true;
    const char* base = reinterpret_cast<const char*>(c.peers[r]);
    const char* q = reinterpret_cast<const char*>(p);
    if (q >= base && q + bytes <= base + c.debug_extent) return true;
    report(c.status, kBadPeerAccess, c.rank, r, detail);
    return false;
}

__device__ __forceinline__ bool wait_ge_sys(const uint64_t* flag, uint64_t want, long long limit) {
    if (ld_acquire_sys(flag) >= want) return true;
    const long long t0 = clock64();
    while (ld_acquire_sys(flag) < want) {
        if (clock64() - t0 > limit) return false;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// warp helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int lane_id() {
    int l;
    asm("mov.s32 %0, %%laneid;" : "=r"(l));
    return l;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_incl_scan(int v) {
    const int l = lane_id();
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, o);
        if (l >= o) v += n;
    }
    return v;
}

// ---------------------------------------------------------------------------------------------
// FP8 e4m3 block scaling (128 channels per scale).  amax is clamped to 1e-4, scale = amax / 448,
// optionally rounded up to a power of two; same math as the reference's per_token_cast_to_fp8
// (csrc/kernels/efa_kernels.cu:143-163) and tests/utils.py:50-58.
// ---------------------------------------------------------------------------------------------
constexpr float kFp8Max = 448.0f;
constexpr float kFp8AmaxFloor = 1e-4f;

__device__ __forceinline__ void fp8_scale_from_amax(float amax, bool round_pow2, float& scale, float& inv_scale) {
    amax = fmaxf(amax, kFp8AmaxFloor);
    if (round_pow2) {
        // smallest power of two >= amax/448
        const float s = amax / kFp8Max;
        int e;
        const float m = frexpf(s, &e);           // s = m * 2^e, m in [0.5,1)
        scale = ldexpf(1.0f, (m == 0.5f) ? e - 1 : e);
        inv_scale = 1.0f / scale;
    } else {
        scale = amax / kFp8Max;
        // 448 * (1 / amax), not 448 / amax: this is what `448.0 / tensor` evaluates to in PyTorch, and the
        // one-ulp difference decides ties when rounding to e4m3.
        inv_scale = kFp8Max * __frcp_rn(amax);
    }
}

// Packs four floats into four e4m3 bytes (round-to-nearest-even, saturating).
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t v) {
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
    return __bfloat1622float2(b);
}
__device__ __forceinline__ uint32_t f2_to_bf16x2(float a, float b) {
    __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Sequence numbers live on the device, one per kernel family, so that a launch carries no
// call-specific argument and can be replayed from a CUDA graph. Every CTA of a launch reads
// `last + 1` when it starts; the last CTA to finish (see cta_is_last) stores the new value. All ranks
// run the same order of collective kernels, so their counters move in lock-step.

__device__ __forceinline__ uint64_t next_seq(const RankCtx& c, int fam) {
    return *reinterpret_cast<volatile uint64_t*>(c.seq + fam) + 1;
}
__device__ __forceinline__ void commit_seq(const RankCtx& c, int fam, uint64_t seq) {
    *reinterpret_cast<volatile uint64_t*>(c.seq + fam) = seq;
}

// Programmatic dependent launch: wait until the predecessor kernel in the stream has completed (and its memory is
// visible), and allow the successor's launch to be prepared. Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_wait_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_successor() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Phase time stamp (nanoseconds of the GPU's global timer) for the tracing facility; free when tracing is off.
__device__ __forceinline__ void trace_stamp(const RankCtx& c, int fam, int slot, int idx) {
    if (c.trace != nullptr && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        c.trace[(fam * 2 + slot) * kTraceStampsPerSlot + idx] = t;
    }
}

// Posts `n` payload words + a sequence number into `dst`'s mailbox slot [kind][me]. One thread.
__device__ __forceinline__ void mailbox_post(const RankCtx& c, int kind, int dst, const uint64_t* words, int n, uint64_t seq) {
    Mailbox* mb = &c.ctrl(dst)->mailbox[kind][c.rank];
    for (int i = 0; i < n; ++i) st_relaxed_sys(&mb->payload[i], words[i]);
    st_release_sys(&mb->seq, seq);
}
// Waits for the slot [kind][src] of my own mailbox to reach `seq`, then copies the payload out.
__device__ __forceinline__ bool mailbox_wait(const RankCtx& c, int kind, int src, uint64_t seq, uint64_t* words, int n) {
    Mailbox* mb = &c.my_ctrl()->mailbox[kind][src];
    if (!wait_ge_sys(&mb->seq, seq, c.timeout_cycles)) return false;
    for (int i = 0; i < n; ++i) words[i] = ld_relaxed_sys(&mb->payload[i]);
    return true;
}

// Cross-rank barrier executed by the first `num_ranks` threads of ONE CTA (call with all threads of
// the CTA; contains __syncthreads). Before it, the CTA's earlier global writes are made visible at
// system scope. Sequence `seq` must be larger than any sequence used before on this Buffer.
// Counterpart of the reference's barrier_block (csrc/kernels/utils.cuh:504-534) without the +-1024
// counter trick and without trap.
enum BarrierKind : int { kBarExplicit = 0, kBarDispatch = 1, kBarCombine = 2, kBarLL = 3 };

__device__ __forceinline__ bool cta_rank_barrier(const RankCtx& c, uint64_t seq) {
    __shared__ int s_ok;
    __syncthreads();  // readers of an earlier call's result are done before the flag is rewritten
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < c.num_ranks) {
        st_release_sys(&c.ctrl(threadIdx.x)->barrier_in[kBarExplicit][c.rank], seq);
        if (!wait_ge_sys(&c.my_ctrl()->barrier_in[kBarExplicit][threadIdx.x], seq, c.timeout_cycles)) {
            report(c.status, kTimeoutBarrier, c.rank, threadIdx.x, (int)seq);
            s_ok = 0;
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// Grid-wide "everyone is done" detection for one rank's slice of a launch (gridDim.x CTAs).
// Returns true in exactly one CTA: the last one to arrive. `ticket` is zero between kernels.
__device__ __forceinline__ bool cta_is_last(int* ticket, int num_ctas) {
    // GPU scope is enough: the ticket is rank-local. A caller that publishes to peers afterwards does so
    // with a system-scope release, which is cumulative over everything ordered before it here.
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_acq_rel_gpu();
        const int old = atomicAdd(ticket, 1);
        s_last = (old == num_ctas - 1);
        if (s_last) {
            *ticket = 0;
            fence_acq_rel_gpu();
        }
    }
    __syncthreads();
    return s_last != 0;
}

}  // namespace dx
