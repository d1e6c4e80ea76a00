// Tuning configuration, buffer-size hints and the low-latency symmetric layout. Host-only, no CUDA
// calls, so it is unit-tested on a machine without a GPU.
//
// `Config` keeps the five-integer signature of the reference (csrc/config.hpp:23-50) so that code
// written against it keeps working. In this design only `num_sms` selects anything (the grid size of
// the dispatch / combine kernels); the four chunk sizes described ring queues that do not exist here
// and are validated and stored only.
//
// Size hints: the reference sizes ring queues (csrc/config.hpp:52-74). Here the symmetric buffer holds
// a fixed control block plus an arena from which the FINAL output tensors are carved, so the hint is
// control block + room for the outputs of `kArenaDepth` dispatches of `max_tokens` tokens per rank
// when every token goes to every rank.
#pragma once

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace dxh {

inline uint64_t align_up(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }

constexpr uint64_t kControlBytes = 1ull << 20;   // control block lives in the first MiB
constexpr uint64_t kBufferAlign = 128;           // same alignment as the reference (configs.cuh)
constexpr int kDefaultHintTokens = 4096;         // tokens per rank assumed by get_nvl_buffer_size_hint
constexpr int kArenaDepth = 4;                   // live dispatch results the default hint leaves room for

struct Config {
    int num_sms;
    int num_max_nvl_chunked_send_tokens;
    int num_max_nvl_chunked_recv_tokens;
    int num_max_rdma_chunked_send_tokens;
    int num_max_rdma_chunked_recv_tokens;

    Config(int sms = 32, int nvl_send = 6, int nvl_recv = 256, int rdma_send = 6, int rdma_recv = 256)
        : num_sms(sms),
          num_max_nvl_chunked_send_tokens(nvl_send),
          num_max_nvl_chunked_recv_tokens(nvl_recv),
          num_max_rdma_chunked_send_tokens(rdma_send),
          num_max_rdma_chunked_recv_tokens(rdma_recv) {
        if (num_sms < 0) throw std::invalid_argument("Config: num_sms must be >= 0");
        if (nvl_send <= 0 || nvl_recv <= 0 || nvl_send >= nvl_recv)
            throw std::invalid_argument("Config: need 0 < nvl_send < nvl_recv");
        if (rdma_send <= 0 || rdma_recv <= 0) throw std::invalid_argument("Config: RDMA chunk sizes must be > 0");
        num_max_rdma_chunked_recv_tokens = (int)align_up(rdma_recv, rdma_send);
        if (rdma_send > num_max_rdma_chunked_recv_tokens / 2)
            throw std::invalid_argument("Config: rdma_send must be <= rdma_recv / 2");
    }

    // Bytes one dispatch result takes in the arena when `rows` rows arrive.
    static uint64_t dispatch_result_bytes(uint64_t rows, uint64_t hidden_bytes, int num_topk, int num_scales) {
        uint64_t b = 0;
        b += align_up(rows * hidden_bytes, 1024);
        b += align_up(rows * (uint64_t)num_scales * 4, 1024);
        b += align_up(rows * (uint64_t)num_topk * 8, 1024);
        b += align_up(rows * (uint64_t)num_topk * 4, 1024);
        b += align_up(rows * 4, 1024);
        return b;
    }

    uint64_t get_nvl_buffer_size_hint(uint64_t hidden_bytes, int num_ranks, int max_tokens_per_rank = kDefaultHintTokens) const {
        if (num_ranks < 1) throw std::invalid_argument("num_ranks must be >= 1");
        const uint64_t rows = (uint64_t)max_tokens_per_rank * (uint64_t)num_ranks;  // every token to every rank
        // payload + a BF16 combine input of the same shape
        const uint64_t one = dispatch_result_bytes(rows, hidden_bytes, 128, 128) + align_up(rows * hidden_bytes, 1024);
        return align_up(kControlBytes + one * kArenaDepth, kBufferAlign);
    }

    // Multi-node (RDMA) transport is a stub on a single NVSwitch box: nothing to reserve.
    uint64_t get_rdma_buffer_size_hint(int64_t /*hidden_bytes*/, int /*num_ranks*/) const { return 0; }
};

// Low-latency symmetric region. Everything a peer writes into lands at the same offset on every rank.
// Two parities (call sequence odd/even) so that call n+1 may start while slow ranks still read call n.
//
//   counts        int  [R][E]             rows each source sends to each expert (all-gathered)
//   recv_x        u8   [L][N][hidden*eb]  dispatch landing zone; IS packed_recv_x (no unpack pass)
//   recv_scales   f32  [L][N][hidden/128]
//   recv_src_info i32  [L][N]
//   combine_stage bf16 [E][max_tokens][hidden]   rows pushed back to the token's home rank
//   combine_src   bf16 [L][N][hidden]     buffer handed out by get_next_low_latency_combine_buffer
// with N = R * max_tokens, L = E / R.
//
// The reference lays out send / recv / signalling areas for RDMA messages
// (csrc/config.hpp:127-187: dispatch msg = 16 + max(2*hidden, hidden + 4*scales) bytes); here there
// are no send buffers at all because senders store straight from registers into the peer.
struct LowLatencyLayout {
    uint64_t counts_off[2], recv_x_off[2], recv_scales_off[2], recv_src_info_off[2], combine_stage_off[2],
        combine_src_off[2];
    uint64_t total_bytes = 0;

    LowLatencyLayout(uint64_t base, int max_tokens, int hidden, int num_ranks, int num_experts) {
        if (num_experts % num_ranks != 0) throw std::invalid_argument("num_experts must be divisible by num_ranks");
        if (hidden % 128 != 0) throw std::invalid_argument("hidden must be a multiple of 128");
        const uint64_t L = num_experts / num_ranks, N = (uint64_t)num_ranks * max_tokens;
        uint64_t off = base;
        auto take = [&](uint64_t bytes) {
            const uint64_t o = off;
            off = align_up(off + bytes, 1024);
            return o;
        };
        for (int p = 0; p < 2; ++p) {
            counts_off[p] = take((uint64_t)num_ranks * num_experts * 4);
            recv_x_off[p] = take(L * N * (uint64_t)hidden * 2);  // sized for BF16 dispatch
            recv_scales_off[p] = take(L * N * (uint64_t)(hidden / 128) * 4);
            recv_src_info_off[p] = take(L * N * 4);
            combine_stage_off[p] = take((uint64_t)num_experts * max_tokens * hidden * 2);
            combine_src_off[p] = take(L * N * (uint64_t)hidden * 2);
        }
        total_bytes = off - base;
    }
};

inline uint64_t get_low_latency_rdma_size_hint(int max_tokens, int hidden, int num_ranks, int num_experts) {
    const uint64_t b = kControlBytes + LowLatencyLayout(0, max_tokens, hidden, num_ranks, num_experts).total_bytes;
    return align_up(b, kBufferAlign);
}

}  // namespace dxh
