// Host side of the cache manager: which pages and which state slot each live
// request holds.
//
// Layers with the same need form a group, and a group has a page pool and a
// block table per request of its own: a group that keeps every key, a group
// that keeps only a window of them. One page id of a group stands for that
// page in every layer of the group. Beside the pages a request holds one slot
// of fixed-size state. The reference's PageTable
// (crates/cellm-cache/src/pagetable.rs:8-122) is the per-request block list of
// one such group; it frees only on cancel (crates/cellm-sdk/src/lib.rs:401-403),
// here pages also go back when a window has passed them.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <vector>

#include "block_allocator.h"

namespace cellm {

struct GroupSpec {
    int num_pages;
    int window;  // 0: every key is kept; w > 0: a token reads only the last w keys (itself included)
};

struct RequestCache {
    int slot = -1;
    int tokens = 0;                               // tokens whose keys are in the cache
    int reserved = 0;                             // tokens that pages have been reserved for
    std::vector<std::vector<int32_t>> blocks;     // per group: page of block i, or -1 once released
    std::vector<int> first_live;                  // per group: first block not yet released
};

class CacheManager {
public:
    CacheManager(int page_size, std::vector<GroupSpec> groups, int num_slots);

    int page_size() const { return page_size_; }
    int num_groups() const { return (int)groups_.size(); }
    const GroupSpec& group(int g) const { return groups_.at((size_t)g); }
    int free_pages(int g) const { return allocs_.at((size_t)g)->free_count(); }
    int free_slots() const { return slots_.free_count(); }
    int num_slots() const { return slots_.total(); }
    int live_requests() const { return (int)requests_.size(); }
    bool has(int64_t id) const { return requests_.count(id) != 0; }

    // Takes a state slot for a new request; returns it, or -1 when none is free.
    int add_request(int64_t id);
    // New pages each group needs so that the request can hold `new_total` tokens.
    std::vector<int> pages_needed(int64_t id, int new_total) const;
    bool can_reserve(int64_t id, int new_total) const;
    // Whether the free pages suffice for the most pages the request holds at any time while it grows to
    // `tokens` tokens in portions of at most `portion`: all of them in a group that keeps every key,
    // the window and one portion in a windowed group (pages_for), less what it holds already.
    bool can_hold(int64_t id, int tokens, int portion) const;
    // Reserves pages in every group for tokens up to new_total; all or nothing.
    bool reserve(int64_t id, int new_total);
    // Marks tokens up to new_total as written and gives back the pages of
    // windowed groups that no later token can read.
    void commit(int64_t id, int new_total);
    // Gives back all pages and the slot.
    void release(int64_t id);

    const RequestCache& request(int64_t id) const;
    // Smallest number of pages group g must have so that a lone request of
    // `tokens` tokens, fed in portions of at most `portion`, always fits.
    int pages_for(int g, int tokens, int portion) const;

private:
    int blocks_for(int tokens) const { return (tokens + page_size_ - 1) / page_size_; }
    int page_size_;
    std::vector<GroupSpec> groups_;
    std::vector<std::unique_ptr<BlockAllocator>> allocs_;
    SlotPool slots_;
    std::map<int64_t, RequestCache> requests_;
};

}  // namespace cellm
