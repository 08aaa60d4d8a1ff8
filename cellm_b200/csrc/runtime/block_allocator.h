// Page allocator of the cache manager.
//
// Same contract as the reference's BlockAllocator
// (crates/cellm-cache/src/allocator.rs:11-90): page ids 0..n-1, a FIFO free
// list so that a freed page goes to the back and is handed out again only
// after the pages freed before it, an all-or-nothing alloc_n, and errors for a
// double free or an id out of range.
#pragma once
#include <cstdint>
#include <deque>
#include <stdexcept>
#include <string>
#include <vector>

namespace cellm {

struct CacheError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class BlockAllocator {
public:
    explicit BlockAllocator(int total);
    int total() const { return total_; }
    int free_count() const { return (int)free_.size(); }
    bool is_free(int id) const;
    // One page, or -1 when none is free.
    int alloc();
    // n pages appended to `out`, or false (and nothing taken) when fewer are free.
    bool alloc_n(int n, std::vector<int32_t>& out);
    void free(int id);

private:
    int total_;
    std::deque<int32_t> free_;
    std::vector<uint8_t> is_free_;
};

// Fixed pool of state slots (one per live request).
class SlotPool {
public:
    explicit SlotPool(int total) : alloc_(total) {}
    int total() const { return alloc_.total(); }
    int free_count() const { return alloc_.free_count(); }
    int take() { return alloc_.alloc(); }
    void give_back(int slot) { alloc_.free(slot); }

private:
    BlockAllocator alloc_;
};

}  // namespace cellm
