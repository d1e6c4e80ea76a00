// Plain-data types shared by host code and kernels: limits, status codes, the symmetric control block
// and the per-rank context. Includable from ordinary C++ (no device code outside __CUDACC__ guards).
#pragma once

#include <stdint.h>

namespace dx {

constexpr int kMaxRanks = 8;            // one NVSwitch domain
constexpr int kMaxLocalExperts = 1024;  // same cap as the reference (configs.cuh:6)
constexpr int kMaxTopk = 32;
constexpr int kMaxVirtualRanks = 8;     // ranks emulated inside one launch (single-GPU test mode)
constexpr int kMaxFusedExperts = 2048;  // experts of the whole group in the expert-major (fused MoE) dispatch

// Error codes written to the status word (the host decodes them in csrc/host/runtime.hpp).
enum Status : int {
    kOk = 0,
    kTimeoutBarrier = 1,
    kTimeoutNotify = 2,
    kTimeoutDescriptor = 3,
    kTimeoutLLCount = 4,
    kTimeoutLLData = 5,
    kTimeoutCombineReady = 6,
    kTimeoutCombineData = 7,
    kTimeoutGemm = 8,
    kBadArgument = 9,
    kTimeoutTest = 10,
    kBadPeerAccess = 11,  // debug bounds check: a row address fell outside the peer's symmetric buffer (access skipped)
    kTimeoutFusedNotify = 12,
};

// Written by kernels into mapped pinned host memory; read by the host after collective calls.
struct StatusBlock {
    // Lives in mapped pinned host memory; the host reads it after every collective call.
    int code;      // Status
    int rank;      // who gave up
    int peer;      // on whom
    int detail;    // kernel-specific (channel, expert, phase)
};

// ---------------------------------------------------------------------------------------------
// symmetric control block.  One per rank at offset 0 of its symmetric buffer; every word in it is
// written by a PEER (or by this rank for its own slot) and read only by the owner.
// All sequence numbers grow monotonically for the life of the Buffer, so nothing is ever reset and a
// word that arrives before the owner starts waiting is still seen (the property the reference gets
// from GdrCounter, csrc/transport/gdr_signal.h:139-205).
// ---------------------------------------------------------------------------------------------
constexpr int kNumMailboxKinds = 6;
constexpr int kMailboxWords = 8;
enum MailboxKind : int {
    kMbDispatchDesc = 0,   // receiver -> sender: where to put rows
    kMbCombineSrc = 1,     // expert rank -> home rank: where the rows to pull live
    kMbChanPrefix = 2,     // flag only: channel prefix row arrived
    kMbLLDispatch = 3,
    kMbLLCombine = 4,
    kMbSpare = 5,
};

struct Mailbox {
    uint64_t payload[kMailboxWords - 1];
    uint64_t seq;  // written last, with release
};

constexpr int kMaxChannels = 128;

struct alignas(128) ControlBlock {
    // peer r stores its sequence here; one row per kernel family so that kernels of different
    // families running on different streams cannot satisfy each other's waits
    uint64_t barrier_in[4][kMaxRanks];
    Mailbox mailbox[kNumMailboxKinds][kMaxRanks];          // [kind][source rank]
    // normal-mode notify: row r = what rank r tells me
    uint64_t notify_seq[kMaxRanks];
    int notify_rank_counts[kMaxRanks][kMaxRanks];          // source's whole num_tokens_per_rank[]
    int notify_expert_counts[kMaxRanks][kMaxLocalExperts]; // source's counts for MY local experts
    int chan_prefix_in[kMaxRanks][kMaxChannels];           // source's per-channel prefix towards me
    // low-latency mode, two parities (the count exchange needs no flag here: its words carry their own validity tag)
    uint64_t ll_data_arrived[2][kMaxRanks];                // monotonically growing row counters
    uint64_t ll_combine_arrived[2][kMaxRanks];
    int ll_mask[kMaxRanks];                                // 1 = rank is masked out (shrink mode)
    // pull combine: rank r tells me where its expert outputs lie, (call tag << 40) | byte offset in its symmetric buffer.
    // Two slots, by the parity of the call's sequence number: a combine that overlaps the tail of its dispatch can post for
    // call n+1 while a slower rank has not yet read the word of call n (never further ahead: call n+2 needs that rank's word
    // of call n+1).
    uint64_t ll_pull_src[2][kMaxRanks];
    // expert-major dispatch (fused MoE layer): row r = what rank r tells me
    uint64_t em_seq[kMaxRanks];
    // two parities (call sequence odd / even): a fast rank may start its next exchange while a slow one still reads this one
    uint64_t em_desc[2][kMaxRanks][4];                     // rank r's receive buffers: rows, scales, row info, combine stage (offsets)
    int em_counts[2][kMaxRanks][kMaxFusedExperts];         // rank r's selections per GLOBAL expert (every rank gets the whole vector)
    uint64_t em_arrived[kMaxLocalExperts];                 // rows landed so far per local expert, monotonic; gates the expert GEMM
};

static_assert(sizeof(ControlBlock) <= (1u << 20), "control block must fit the first MiB of the symmetric buffer");

// What every kernel needs to know about "this rank".
struct RankCtx {
    int rank;
    int num_ranks;
    void* peers[kMaxRanks];      // peers[rank] is this rank's own symmetric buffer
    StatusBlock* status;         // mapped host memory
    int* local_scratch;          // small rank-local device scratch (tickets), zero between kernels
    uint64_t* seq;               // rank-local device memory: last finished sequence of every kernel family
    unsigned long long* trace;   // optional device buffer for phase time stamps (nullptr = tracing off)
    long long timeout_cycles;
    int mask_on_timeout;         // low-latency shrink mode: a rank that times out is masked instead of failing the call
    unsigned long long debug_extent;  // 0 = off; else bytes of every rank's symmetric buffer: row addresses are range-checked

#ifdef __CUDACC__
    __device__ __forceinline__ ControlBlock* ctrl(int r) const { return reinterpret_cast<ControlBlock*>(peers[r]); }
    __device__ __forceinline__ ControlBlock* my_ctrl() const { return reinterpret_cast<ControlBlock*>(peers[rank]); }
    template <typename T>
    __device__ __forceinline__ T* at(int r, uint64_t off) const {
        return reinterpret_cast<T*>(reinterpret_cast<char*>(peers[r]) + off);
    }
#endif
};

// Kernel families; each has its own monotonically growing sequence number on every rank.
// Rank-local u64 words behind RankCtx::seq: [kNumFamilies] sequences, [2 kinds][2 parities][kMaxRanks] expected low-latency
// arrivals, [kMaxLocalExperts] expected rows per local expert of the expert-major dispatch.
constexpr int kFusedExpectedWord0 = 8 + 2 * 2 * kMaxRanks;
constexpr int kTraceStampsPerSlot = 16;  // trace layout: [family][slot 0 = first CTA, 1 = last CTA][stamp]

enum Family : int { kFamNotify = 0, kFamDispatch = 1, kFamCombine = 2, kFamBarrier = 3, kFamLLDispatch = 4, kFamLLCombine = 5, kFamFused = 6, kNumFamilies = 8 };
static_assert(kFusedExpectedWord0 == kNumFamilies + 2 * 2 * kMaxRanks, "layout of the rank-local sequence words");
// after the fused layer's expected-arrival words: per parity, the sequence number of the low-latency dispatch that last used it
constexpr int kLLStartedWord0 = kFusedExpectedWord0 + kMaxLocalExperts;

}  // namespace dx
