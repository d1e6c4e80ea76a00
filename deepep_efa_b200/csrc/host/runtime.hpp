// Per-rank host runtime: owns the symmetric buffer (cudaMalloc + CUDA IPC), the arena carved out of
// it, the mapped host words the kernels report through, and the rank-local device state (tickets,
// sequence counters). One instance per rank; a single process may own several (single-GPU emulation
// of a multi-rank job, where "peers" are simply the other instances' buffers).
//
// Reference counterparts: deep_ep::Buffer constructor / sync / destroy (csrc/deep_ep.cpp:206-515),
// SharedMemoryAllocator (csrc/deep_ep.cpp:93-202), mapped counters (csrc/deep_ep.cpp:281-296).
// Differences: no NVSHMEM/EFA state, no workspace, outputs are carved from the symmetric arena, errors
// come back through a status block instead of a device trap.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../kernels/api.h"
#include "arena.hpp"
#include "config.hpp"

namespace dxh {

#define DX_CUDA_CHECK(expr)                                                                              \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess) {                                                                         \
            char _buf[512];                                                                              \
            std::snprintf(_buf, sizeof(_buf), "CUDA error %s (%s) at %s:%d: %s", cudaGetErrorName(_e),   \
                          cudaGetErrorString(_e), __FILE__, __LINE__, #expr);                            \
            cudaGetLastError();                                                                          \
            throw std::runtime_error(_buf);                                                              \
        }                                                                                                \
    } while (0)

inline const char* status_name(int code) {
    switch (code) {
        case dx::kOk: return "ok";
        case dx::kTimeoutBarrier: return "timeout in cross-rank barrier";
        case dx::kTimeoutNotify: return "timeout waiting for token counts (notify)";
        case dx::kTimeoutDescriptor: return "timeout waiting for a peer's receive descriptor";
        case dx::kTimeoutLLCount: return "timeout waiting for low-latency expert counts";
        case dx::kTimeoutLLData: return "timeout waiting for low-latency dispatch rows";
        case dx::kTimeoutCombineReady: return "timeout waiting for a peer's combine source";
        case dx::kTimeoutCombineData: return "timeout waiting for low-latency combine rows";
        case dx::kTimeoutGemm: return "timeout inside grouped GEMM pipeline";
        case dx::kBadArgument: return "kernel rejected its arguments";
        case dx::kTimeoutTest: return "timeout probe (expected in tests)";
        case dx::kTimeoutFusedNotify: return "timeout waiting for expert counts (expert-major dispatch)";
        case dx::kBadPeerAccess: return "debug bounds check: a row address fell outside the peer's symmetric buffer (access skipped)";
        default: return "unknown status";
    }
}

// Host words the device writes; all in one mapped pinned allocation.
struct HostWords {
    dx::StatusBlock status;
    volatile int recv_counter;                         // -1 = not yet, -2 = notify failed
    volatile int expert_counter[dx::kMaxLocalExperts];
};

constexpr int kLocalScratchInts = 64;
// sequences + low-latency expected arrivals + expected rows per local expert of the expert-major dispatch
constexpr int kLocalSeqWords = dx::kLLStartedWord0 + 2;

class RuntimeCore {
  public:
    RuntimeCore(int rank, int num_ranks, uint64_t num_nvl_bytes, uint64_t num_ll_bytes, int device, double timeout_ms,
                bool mask_on_timeout)
        : rank_(rank), num_ranks_(num_ranks), device_(device), mask_on_timeout_(mask_on_timeout) {
        if (num_ranks < 1 || num_ranks > dx::kMaxRanks) throw std::invalid_argument("num_ranks must be in [1, 8]: one NVSwitch domain");
        if (rank < 0 || rank >= num_ranks) throw std::invalid_argument("rank out of range");
        DX_CUDA_CHECK(cudaSetDevice(device_));
        ll_base_ = kControlBytes;
        ll_bytes_ = align_up(num_ll_bytes, 1024);
        const uint64_t arena_base = ll_base_ + ll_bytes_;
        const uint64_t arena_bytes = num_nvl_bytes > kControlBytes ? align_up(num_nvl_bytes - kControlBytes, 1024) : 0;
        total_bytes_ = arena_base + arena_bytes;
        DX_CUDA_CHECK(cudaMalloc(&base_, total_bytes_));
        // control block, and the low-latency region: its count words carry validity tags and must not start with stale ones
        DX_CUDA_CHECK(cudaMemset(base_, 0, kControlBytes + ll_bytes_));
        arena_.reset(arena_base, arena_bytes);
        DX_CUDA_CHECK(cudaMalloc(&local_scratch_, kLocalScratchInts * sizeof(int)));
        DX_CUDA_CHECK(cudaMemset(local_scratch_, 0, kLocalScratchInts * sizeof(int)));
        DX_CUDA_CHECK(cudaMalloc(&local_seq_, kLocalSeqWords * sizeof(uint64_t)));
        DX_CUDA_CHECK(cudaMemset(local_seq_, 0, kLocalSeqWords * sizeof(uint64_t)));
        DX_CUDA_CHECK(cudaMalloc(&never_set_flag_, sizeof(uint64_t)));
        DX_CUDA_CHECK(cudaMemset(never_set_flag_, 0, sizeof(uint64_t)));
        DX_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_), sizeof(HostWords), cudaHostAllocMapped));
        std::memset((void*)host_, 0, sizeof(HostWords));
        host_->recv_counter = -1;
        DX_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev_), (void*)host_, 0));
        int khz = 0;
        DX_CUDA_CHECK(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device_));
        clock_khz_ = khz > 0 ? khz : 1965000;
        set_timeout_ms(timeout_ms);
        if (const char* e = std::getenv("DEEPEP_DEBUG_CHECKS"); e != nullptr && e[0] == '1') debug_checks_ = true;
        for (int i = 0; i < dx::kMaxRanks; ++i) peers_[i] = nullptr;
        peers_[rank_] = base_;
        DX_CUDA_CHECK(cudaDeviceSynchronize());
    }

    ~RuntimeCore() { release(); }

    void set_debug_checks(bool on) { debug_checks_ = on; }
    bool debug_checks() const { return debug_checks_; }
    // Test hook: check row addresses against a smaller extent than the real allocation (0 = the real size), so that a test
    // can provoke a violation with an address that still lies inside this rank's own buffer.
    void set_debug_extent(uint64_t bytes) { debug_extent_override_ = bytes; }

    void set_timeout_ms(double ms) {
        timeout_ms_ = ms;
        timeout_cycles_ = (long long)(ms * (double)clock_khz_);
    }
    double timeout_ms() const { return timeout_ms_; }

    std::string ipc_handle() const {
        cudaIpcMemHandle_t h;
        DX_CUDA_CHECK(cudaIpcGetMemHandle(&h, base_));
        return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
    }

    // Real multi-process bootstrap: handles[r] is rank r's IPC handle, device_ids[r] its CUDA device.
    void open_peers(const std::vector<std::string>& handles) {
        if ((int)handles.size() != num_ranks_) throw std::invalid_argument("open_peers: need one handle per rank");
        DX_CUDA_CHECK(cudaSetDevice(device_));
        for (int r = 0; r < num_ranks_; ++r) {
            if (r == rank_) continue;
            if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("open_peers: bad handle size");
            cudaIpcMemHandle_t h;
            std::memcpy(&h, handles[r].data(), sizeof(h));
            void* p = nullptr;
            DX_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
            peers_[r] = p;
            ipc_opened_[r] = true;
        }
        available_ = true;
    }

    // Single-process emulation: the peers are other RuntimeCore objects on the same device.
    void set_local_peers(const std::vector<RuntimeCore*>& all) {
        if ((int)all.size() != num_ranks_) throw std::invalid_argument("set_local_peers: need one runtime per rank");
        for (int r = 0; r < num_ranks_; ++r) peers_[r] = all[r]->base_;
        available_ = true;
    }

    void release() {
        if (released_) return;
        released_ = true;
        cudaSetDevice(device_);
        cudaDeviceSynchronize();
        drain_pending(true);
        for (int r = 0; r < num_ranks_; ++r)
            if (ipc_opened_[r]) cudaIpcCloseMemHandle(peers_[r]);
        if (base_) cudaFree(base_);
        if (local_scratch_) cudaFree(local_scratch_);
        if (local_seq_) cudaFree(local_seq_);
        if (never_set_flag_) cudaFree(never_set_flag_);
        if (trace_) cudaFree(trace_);
        trace_ = nullptr;
        if (host_) cudaFreeHost((void*)host_);
        base_ = nullptr;
        available_ = false;
    }

    dx::RankCtx ctx() const {
        dx::RankCtx c;
        c.rank = rank_;
        c.num_ranks = num_ranks_;
        for (int i = 0; i < dx::kMaxRanks; ++i) c.peers[i] = peers_[i];
        c.status = &host_dev_->status;
        c.local_scratch = local_scratch_;
        c.seq = local_seq_;
        c.trace = trace_;
        c.timeout_cycles = timeout_cycles_;
        c.mask_on_timeout = mask_on_timeout_ ? 1 : 0;
        c.debug_extent = debug_checks_ ? (unsigned long long)(debug_extent_override_ != 0 ? debug_extent_override_ : total_bytes_) : 0ull;
        return c;
    }

    // ---- arena ------------------------------------------------------------------------------
    // Returns the offset of a fresh block. Blocks released earlier become reusable once the streams
    // that may still touch them have passed the events recorded at release time.
    uint64_t arena_alloc(uint64_t bytes) {
        std::lock_guard<std::mutex> g(mu_);
        drain_pending(false);
        int64_t off = arena_.alloc(bytes);
        if (off < 0) {
            drain_pending(true);
            off = arena_.alloc(bytes);
        }
        if (off < 0) {
            char buf[512];
            std::snprintf(buf, sizeof(buf),
                          "symmetric arena exhausted: need %llu B, capacity %llu B, in use %llu B, largest free block %llu B. "
                          "Create the Buffer with a larger num_nvl_bytes (Config.get_nvl_buffer_size_hint) or drop references "
                          "to earlier dispatch results.",
                          (unsigned long long)bytes, (unsigned long long)arena_.capacity(), (unsigned long long)arena_.in_use(),
                          (unsigned long long)arena_.largest_free());
            throw std::runtime_error(buf);
        }
        return (uint64_t)off;
    }

    // Called from tensor deleters (any thread). `streams` are streams whose queued work may still
    // use the block.
    void arena_release(uint64_t off, const std::vector<cudaStream_t>& streams) {
        std::lock_guard<std::mutex> g(mu_);
        if (released_) return;
        Pending p;
        p.off = off;
        int prev = -1;
        cudaGetDevice(&prev);
        if (prev != device_) cudaSetDevice(device_);
        for (cudaStream_t s : streams) {
            cudaEvent_t ev = nullptr;
            if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
                if (cudaEventRecord(ev, s) == cudaSuccess) p.events.push_back(ev);
                else cudaEventDestroy(ev);
            }
        }
        cudaGetLastError();
        if (prev != device_ && prev >= 0) cudaSetDevice(prev);
        pending_.push_back(std::move(p));
    }

    bool in_symmetric(const void* p, uint64_t bytes, uint64_t* off) const {
        const char* b = reinterpret_cast<const char*>(base_);
        const char* q = reinterpret_cast<const char*>(p);
        if (q < b || q + bytes > b + total_bytes_) return false;
        *off = (uint64_t)(q - b);
        return true;
    }

    // ---- host <-> device words ----------------------------------------------------------------
    void reset_recv_counters(int num_local_experts) {
        host_->recv_counter = -1;
        for (int i = 0; i < num_local_experts; ++i) host_->expert_counter[i] = -1;
    }

    // Spins until the notify kernel has published the receive counts. Bounded by the host timeout.
    int wait_recv_counts(int num_local_experts, std::vector<int>* per_expert) {
        const auto t0 = std::chrono::steady_clock::now();
        const double limit_ms = timeout_ms_ * 2 + 1000.0;
        while (true) {
            const int n = host_->recv_counter;
            bool ready = n >= 0;
            if (n == -2) raise_status("dispatch");
            if (ready)
                for (int i = 0; i < num_local_experts; ++i) ready = ready && host_->expert_counter[i] >= 0;
            if (ready) {
                per_expert->resize(num_local_experts);
                for (int i = 0; i < num_local_experts; ++i) (*per_expert)[i] = host_->expert_counter[i];
                return n;
            }
            const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            if (ms > limit_ms) {
                if (host_->status.code != 0) raise_status("dispatch");
                throw std::runtime_error("dispatch: host timed out waiting for the receive counts (did every rank call dispatch?)");
            }
        }
    }

    // ---- tracing -------------------------------------------------------------------------------
    // Kernels stamp the GPU global timer at phase boundaries of their first and last CTA.
    void enable_trace(bool on) {
        DX_CUDA_CHECK(cudaSetDevice(device_));
        if (on && trace_ == nullptr) {
            DX_CUDA_CHECK(cudaMalloc(&trace_, kTraceWords * sizeof(unsigned long long)));
            DX_CUDA_CHECK(cudaMemset(trace_, 0, kTraceWords * sizeof(unsigned long long)));
        } else if (!on && trace_ != nullptr) {
            DX_CUDA_CHECK(cudaDeviceSynchronize());
            cudaFree(trace_);
            trace_ = nullptr;
        }
    }
    std::vector<unsigned long long> read_trace() {
        std::vector<unsigned long long> v(kTraceWords, 0);
        if (trace_ != nullptr) {
            DX_CUDA_CHECK(cudaSetDevice(device_));
            DX_CUDA_CHECK(cudaDeviceSynchronize());
            DX_CUDA_CHECK(cudaMemcpy(v.data(), trace_, kTraceWords * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        }
        return v;
    }

    int status_code() const { return read_word(&host_->status.code); }
    std::string status_string() const {
        const int code = read_word(&host_->status.code), rank = read_word(&host_->status.rank);
        const int peer = read_word(&host_->status.peer), detail = read_word(&host_->status.detail);
        char buf[256];
        std::snprintf(buf, sizeof(buf), "%s [code %d, rank %d, peer %d, detail %d]", status_name(code), code, rank, peer, detail);
        return std::string(buf);
    }
    void clear_status() { std::memset((void*)&host_->status, 0, sizeof(dx::StatusBlock)); }
    void raise_status(const char* where) {
        std::string m = std::string(where) + ": " + status_string();
        throw std::runtime_error("EPTimeoutError: " + m);
    }

    // Zeroes the control block and the rank-local sequence state. Call on every rank, between two
    // host-level barriers, with no kernel of this Buffer in flight.
    void reset_control() {
        DX_CUDA_CHECK(cudaSetDevice(device_));
        DX_CUDA_CHECK(cudaDeviceSynchronize());
        DX_CUDA_CHECK(cudaMemset(base_, 0, kControlBytes + ll_bytes_));  // sequences restart, so no tagged count word may survive
        DX_CUDA_CHECK(cudaMemset(local_scratch_, 0, kLocalScratchInts * sizeof(int)));
        DX_CUDA_CHECK(cudaMemset(local_seq_, 0, kLocalSeqWords * sizeof(uint64_t)));
        DX_CUDA_CHECK(cudaDeviceSynchronize());
        clear_status();
    }

    int rank() const { return rank_; }
    int num_ranks() const { return num_ranks_; }
    int device() const { return device_; }
    bool available() const { return available_; }
    void* base() const { return base_; }
    uint64_t total_bytes() const { return total_bytes_; }
    uint64_t ll_base() const { return ll_base_; }
    uint64_t ll_bytes() const { return ll_bytes_; }
    const Arena& arena() const { return arena_; }
    uint64_t* never_set_flag() const { return never_set_flag_; }
    uint64_t* local_seq() const { return local_seq_; }
    dx::ControlBlock* control() const { return reinterpret_cast<dx::ControlBlock*>(base_); }

  private:
    static int read_word(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

    struct Pending {
        uint64_t off;
        std::vector<cudaEvent_t> events;
    };

    void drain_pending(bool wait) {
        for (auto it = pending_.begin(); it != pending_.end();) {
            bool done = true;
            for (cudaEvent_t ev : it->events) {
                cudaError_t e = wait ? cudaEventSynchronize(ev) : cudaEventQuery(ev);
                if (e == cudaErrorNotReady) {
                    done = false;
                    break;
                }
            }
            if (done) {
                for (cudaEvent_t ev : it->events) cudaEventDestroy(ev);
                arena_.free(it->off);
                it = pending_.erase(it);
            } else {
                ++it;
            }
        }
        cudaGetLastError();
    }

    int rank_, num_ranks_, device_;
    bool mask_on_timeout_ = false;
    uint64_t debug_extent_override_ = 0;
    bool debug_checks_ = false;  // range-check row addresses on the device (env DEEPEP_DEBUG_CHECKS=1 or set_debug_checks)
    bool available_ = false, released_ = false;
    void* base_ = nullptr;
    uint64_t total_bytes_ = 0, ll_base_ = 0, ll_bytes_ = 0;
    void* peers_[dx::kMaxRanks];
    bool ipc_opened_[dx::kMaxRanks] = {false, false, false, false, false, false, false, false};
    int* local_scratch_ = nullptr;
    uint64_t* local_seq_ = nullptr;
    uint64_t* never_set_flag_ = nullptr;
    unsigned long long* trace_ = nullptr;
    static constexpr int kTraceWords = dx::kNumFamilies * 2 * dx::kTraceStampsPerSlot;
    HostWords* host_ = nullptr;
    HostWords* host_dev_ = nullptr;
    int clock_khz_ = 1965000;
    double timeout_ms_ = 10000.0;
    long long timeout_cycles_ = 0;
    Arena arena_;
    std::deque<Pending> pending_;
    std::mutex mu_;
};

}  // namespace dxh
