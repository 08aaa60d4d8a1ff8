#include "cache_manager.h"

#include <algorithm>
#include <string>

namespace cellm {

CacheManager::CacheManager(int page_size, std::vector<GroupSpec> groups, int num_slots)
    : page_size_(page_size), groups_(std::move(groups)), slots_(num_slots) {
    if (page_size <= 0) throw CacheError("cache: page size must be positive");
    for (const auto& g : groups_) {
        if (g.window < 0) throw CacheError("cache: a window must not be negative");
        allocs_.push_back(std::make_unique<BlockAllocator>(g.num_pages));
    }
}

int CacheManager::add_request(int64_t id) {
    if (requests_.count(id)) throw CacheError("cache: request " + std::to_string(id) + " is already live");
    const int slot = slots_.take();
    if (slot < 0) return -1;
    RequestCache rc;
    rc.slot = slot;
    rc.blocks.resize(groups_.size());
    rc.first_live.assign(groups_.size(), 0);
    requests_.emplace(id, std::move(rc));
    return slot;
}

const RequestCache& CacheManager::request(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw CacheError("cache: request " + std::to_string(id) + " is not live");
    return it->second;
}

std::vector<int> CacheManager::pages_needed(int64_t id, int new_total) const {
    const RequestCache& rc = request(id);
    std::vector<int> need(groups_.size(), 0);
    const int want = blocks_for(new_total);
    for (size_t g = 0; g < groups_.size(); ++g) need[g] = std::max(0, want - (int)rc.blocks[g].size());
    return need;
}

bool CacheManager::can_reserve(int64_t id, int new_total) const {
    const auto need = pages_needed(id, new_total);
    for (size_t g = 0; g < groups_.size(); ++g)
        if (need[g] > allocs_[g]->free_count()) return false;
    return true;
}

bool CacheManager::can_hold(int64_t id, int tokens, int portion) const {
    const RequestCache& rc = request(id);
    for (size_t g = 0; g < groups_.size(); ++g) {
        int held = 0;
        for (int32_t p : rc.blocks[g]) held += p >= 0 ? 1 : 0;
        if (pages_for((int)g, tokens, portion) - held > allocs_[g]->free_count()) return false;
    }
    return true;
}

bool CacheManager::reserve(int64_t id, int new_total) {
    if (!can_reserve(id, new_total)) return false;
    RequestCache& rc = requests_.at(id);
    if (new_total < rc.tokens) throw CacheError("cache: reserve below the tokens already written");
    const auto need = pages_needed(id, new_total);
    for (size_t g = 0; g < groups_.size(); ++g) allocs_[g]->alloc_n(need[g], rc.blocks[g]);
    rc.reserved = std::max(rc.reserved, new_total);
    return true;
}

void CacheManager::commit(int64_t id, int new_total) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw CacheError("cache: request " + std::to_string(id) + " is not live");
    RequestCache& rc = it->second;
    if (new_total < rc.tokens) throw CacheError("cache: commit would shrink request " + std::to_string(id));
    if (new_total > rc.reserved)
        throw CacheError("cache: commit of " + std::to_string(new_total) + " tokens, but pages are reserved for " +
                         std::to_string(rc.reserved));
    rc.tokens = new_total;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int w = groups_[g].window;
        if (w <= 0) continue;
        // The next token sits at position >= tokens and reads keys >= tokens - w + 1.
        const int first_key = rc.tokens - w + 1;
        while (rc.first_live[g] < (int)rc.blocks[g].size() &&
               (rc.first_live[g] + 1) * page_size_ <= first_key) {
            int32_t& p = rc.blocks[g][(size_t)rc.first_live[g]];
            if (p >= 0) allocs_[g]->free(p);
            p = -1;
            ++rc.first_live[g];
        }
    }
}

void CacheManager::release(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw CacheError("cache: request " + std::to_string(id) + " is not live");
    RequestCache& rc = it->second;
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int32_t p : rc.blocks[g])
            if (p >= 0) allocs_[g]->free(p);
    slots_.give_back(rc.slot);
    requests_.erase(it);
}

int CacheManager::pages_for(int g, int tokens, int portion) const {
    const int w = groups_.at((size_t)g).window;
    if (w <= 0) return blocks_for(tokens);
    // Live keys span at most window - 1 earlier keys plus one portion, and may
    // straddle page edges at both ends.
    const int span = std::min(tokens, w - 1 + std::max(1, portion));
    return std::min(blocks_for(tokens), blocks_for(span) + 1);
}

}  // namespace cellm
