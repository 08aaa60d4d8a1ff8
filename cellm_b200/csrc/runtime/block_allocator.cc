#include "block_allocator.h"

namespace cellm {

BlockAllocator::BlockAllocator(int total) : total_(total), is_free_((size_t)(total > 0 ? total : 0), 1) {
    if (total <= 0) throw CacheError("allocator: the number of pages must be positive, got " + std::to_string(total));
    for (int i = 0; i < total; ++i) free_.push_back(i);
}

bool BlockAllocator::is_free(int id) const {
    if (id < 0 || id >= total_) throw CacheError("allocator: page id " + std::to_string(id) + " out of range 0.." + std::to_string(total_ - 1));
    return is_free_[(size_t)id] != 0;
}

int BlockAllocator::alloc() {
    if (free_.empty()) return -1;
    const int id = free_.front();
    free_.pop_front();
    is_free_[(size_t)id] = 0;
    return id;
}

bool BlockAllocator::alloc_n(int n, std::vector<int32_t>& out) {
    if (n < 0) throw CacheError("allocator: alloc_n of a negative count");
    if ((int)free_.size() < n) return false;
    for (int i = 0; i < n; ++i) out.push_back(alloc());
    return true;
}

void BlockAllocator::free(int id) {
    if (id < 0 || id >= total_) throw CacheError("allocator: free of page id " + std::to_string(id) + " out of range 0.." + std::to_string(total_ - 1));
    if (is_free_[(size_t)id]) throw CacheError("allocator: page " + std::to_string(id) + " freed twice");
    is_free_[(size_t)id] = 1;
    free_.push_back(id);
}

}  // namespace cellm
