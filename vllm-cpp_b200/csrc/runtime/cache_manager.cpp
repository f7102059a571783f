#include "cache_manager.h"

#include <algorithm>

namespace vcb {

static inline int32_t ceil_div(int32_t a, int32_t b) { return (a + b - 1) / b; }

IdPool::IdPool(int32_t n) : held_(std::max(n, 0), 0) {
    if (n < 0) throw CacheError("pool size must be >= 0");
    free_.reserve(n);
    // ids are handed out in ascending order from a fresh pool
    for (int32_t i = n - 1; i >= 0; --i) free_.push_back(i);
}

bool IdPool::alloc(int32_t n, std::vector<int32_t>& out) {
    if (n < 0) throw CacheError("alloc of a negative count");
    if ((int32_t)free_.size() < n) return false;
    for (int32_t i = 0; i < n; ++i) {
        const int32_t id = free_.back();
        free_.pop_back();
        held_[id] = 1;
        out.push_back(id);
    }
    return true;
}

void IdPool::free(int32_t id) {
    if (id < 0 || id >= size()) throw CacheError("free of id " + std::to_string(id) + " outside the pool");
    if (!held_[id]) throw CacheError("id " + std::to_string(id) + " freed twice");
    held_[id] = 0;
    free_.push_back(id);
}

CacheManager::CacheManager(std::vector<GroupSpec> groups, int32_t num_slots)
    : groups_(std::move(groups)), slots_(num_slots) {
    for (const auto& g : groups_) {
        if (g.page_size < 1) throw CacheError("page_size must be >= 1");
        if (g.window < 0) throw CacheError("window must be >= 0");
        pools_.emplace_back(g.num_pages);
    }
}

const CacheManager::Seq& CacheManager::seq(int64_t request) const {
    auto it = seqs_.find(request);
    if (it == seqs_.end()) throw CacheError("request " + std::to_string(request) + " is not open");
    return it->second;
}
CacheManager::Seq& CacheManager::seq(int64_t request) {
    auto it = seqs_.find(request);
    if (it == seqs_.end()) throw CacheError("request " + std::to_string(request) + " is not open");
    return it->second;
}

int32_t CacheManager::open(int64_t request) {
    if (seqs_.count(request)) throw CacheError("request " + std::to_string(request) + " is already open");
    std::vector<int32_t> s;
    if (!slots_.alloc(1, s)) return -1;
    Seq q;
    q.slot = s[0];
    q.tables.resize(groups_.size());
    seqs_.emplace(request, std::move(q));
    return s[0];
}

int32_t CacheManager::pages_missing(int64_t request, int32_t group, int32_t new_len) const {
    const GroupSpec& g = groups_.at(group);
    int32_t have = 0;
    if (request >= 0) {
        auto it = seqs_.find(request);
        if (it != seqs_.end()) have = (int32_t)it->second.tables[group].size();
    }
    return std::max(0, ceil_div(new_len, g.page_size) - have);
}

int32_t CacheManager::peak_pages(int32_t group, int32_t total_len, int32_t portion) const {
    const GroupSpec& g = groups_.at(group);
    const int32_t all = ceil_div(total_len, g.page_size);
    if (g.window == 0) return all;
    // a window group holds at most the window, one portion being written and a page of slack at each end
    return std::min(all, ceil_div(g.window + std::max(portion, 1), g.page_size) + 1);
}

bool CacheManager::reserve(int64_t request, int32_t new_len) {
    Seq& q = seq(request);
    if (new_len < q.committed) throw CacheError("reserve below the committed length");
    for (size_t g = 0; g < groups_.size(); ++g)
        if (pages_missing(request, (int32_t)g, new_len) > pools_[g].free_count()) return false;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int32_t n = pages_missing(request, (int32_t)g, new_len);
        if (!pools_[g].alloc(n, q.tables[g])) throw CacheError("internal: pool shrank during reserve");
    }
    q.reserved = std::max(q.reserved, new_len);
    return true;
}

void CacheManager::commit(int64_t request, int32_t new_len) {
    Seq& q = seq(request);
    if (new_len < q.committed) throw CacheError("commit below the committed length");
    if (new_len > q.reserved) throw CacheError("commit beyond the reserved length");
    q.committed = new_len;
    for (size_t g = 0; g < groups_.size(); ++g) {
        const GroupSpec& spec = groups_[g];
        if (spec.window == 0) continue;
        // the next query sits at position new_len and reads keys >= new_len - W + 1
        const int32_t first_needed = std::max(0, new_len - spec.window + 1);
        const int32_t dead_blocks = std::min<int32_t>(first_needed / spec.page_size, (int32_t)q.tables[g].size());
        for (int32_t b = 0; b < dead_blocks; ++b) {
            int32_t& page = q.tables[g][b];
            if (page >= 0) {
                pools_[g].free(page);
                page = -1;
            }
        }
    }
}

void CacheManager::close(int64_t request) {
    Seq& q = seq(request);
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int32_t page : q.tables[g])
            if (page >= 0) pools_[g].free(page);
    slots_.free(q.slot);
    seqs_.erase(request);
}

const std::vector<int32_t>& CacheManager::block_table(int64_t request, int32_t group) const {
    return seq(request).tables.at(group);
}

void CacheManager::check_invariants() const {
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int32_t> owners(pools_[g].size(), 0);
        for (const auto& kv : seqs_)
            for (int32_t page : kv.second.tables[g])
                if (page >= 0) {
                    if (page >= pools_[g].size()) throw CacheError("a block table names a page outside its pool");
                    owners[page]++;
                }
        int32_t held = 0;
        for (int32_t p = 0; p < pools_[g].size(); ++p) {
            if (owners[p] > 1) throw CacheError("page " + std::to_string(p) + " is held twice");
            if (owners[p] == 1 && !pools_[g].is_held(p)) throw CacheError("page " + std::to_string(p) + " is in a table but free");
            if (owners[p] == 0 && pools_[g].is_held(p)) throw CacheError("page " + std::to_string(p) + " is lost (held by no request)");
            held += owners[p];
        }
        if (held + pools_[g].free_count() != pools_[g].size()) throw CacheError("page count does not add up");
    }
    std::vector<int32_t> slot_owner(slots_.size(), 0);
    for (const auto& kv : seqs_) {
        const int32_t s = kv.second.slot;
        if (s < 0 || s >= slots_.size() || !slots_.is_held(s)) throw CacheError("a request holds a bad slot");
        if (++slot_owner[s] > 1) throw CacheError("slot " + std::to_string(s) + " is held twice");
    }
    if ((int32_t)seqs_.size() + slots_.free_count() != slots_.size()) throw CacheError("slot count does not add up");
}

}  // namespace vcb
