// Offset allocator for the symmetric arena: the part of a rank's peer-mapped buffer from which
// dispatch outputs and user-requested symmetric tensors are carved. Host-only bookkeeping (no CUDA),
// first-fit with coalescing; blocks are addressed by their byte offset from the buffer base.
//
// The reference has no counterpart: its outputs are ordinary torch tensors filled by a receiver-side
// copy out of ring queues (csrc/deep_ep.cpp:780-801, csrc/kernels/intranode.cu:465-476). Carving the
// final tensors out of peer-mapped memory is what lets senders store into them directly.
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>

namespace dxh {

class Arena {
  public:
    Arena() = default;
    Arena(uint64_t base, uint64_t size, uint64_t align = 1024) { reset(base, size, align); }

    void reset(uint64_t base, uint64_t size, uint64_t align = 1024) {
        align_ = align;
        const uint64_t b = (base + align - 1) / align * align;
        base_ = b;
        size_ = (base + size > b) ? (base + size - b) / align * align : 0;
        free_.clear();
        used_.clear();
        if (size_ > 0) free_[base_] = size_;
        in_use_ = 0;
        high_water_ = 0;
    }

    // Returns the offset of a block of at least `bytes` bytes, or -1 when nothing fits.
    int64_t alloc(uint64_t bytes) {
        const uint64_t need = bytes == 0 ? align_ : (bytes + align_ - 1) / align_ * align_;
        for (auto it = free_.begin(); it != free_.end(); ++it) {
            if (it->second >= need) {
                const uint64_t off = it->first, rest = it->second - need;
                free_.erase(it);
                if (rest > 0) free_[off + need] = rest;
                used_[off] = need;
                in_use_ += need;
                if (in_use_ > high_water_) high_water_ = in_use_;
                return (int64_t)off;
            }
        }
        return -1;
    }

    void free(uint64_t off) {
        auto u = used_.find(off);
        if (u == used_.end()) throw std::runtime_error("Arena::free: offset " + std::to_string(off) + " is not an allocated block");
        uint64_t size = u->second;
        used_.erase(u);
        in_use_ -= size;
        // coalesce with the next and the previous free block
        auto next = free_.lower_bound(off);
        if (next != free_.end() && off + size == next->first) {
            size += next->second;
            next = free_.erase(next);
        }
        if (next != free_.begin()) {
            auto prev = std::prev(next);
            if (prev->first + prev->second == off) {
                prev->second += size;
                return;
            }
        }
        free_[off] = size;
    }

    bool owns(uint64_t off) const { return used_.count(off) != 0; }
    uint64_t base() const { return base_; }
    uint64_t capacity() const { return size_; }
    uint64_t in_use() const { return in_use_; }
    uint64_t high_water() const { return high_water_; }
    size_t num_free_blocks() const { return free_.size(); }
    uint64_t largest_free() const {
        uint64_t m = 0;
        for (auto& kv : free_) m = kv.second > m ? kv.second : m;
        return m;
    }

  private:
    uint64_t base_ = 0, size_ = 0, align_ = 1024, in_use_ = 0, high_water_ = 0;
    std::map<uint64_t, uint64_t> free_;  // offset -> size
    std::map<uint64_t, uint64_t> used_;
};

}  // namespace dxh
