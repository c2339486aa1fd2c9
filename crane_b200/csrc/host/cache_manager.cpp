#include "cache_manager.hpp"

#include <algorithm>

#define CRANE_HOST_API extern "C" __attribute__((visibility("default")))

namespace crane {

CacheManager::CacheManager(const std::vector<GroupSpec>& groups, int max_requests)
    : groups_(groups), max_requests_(max_requests) {
    free_.resize(groups_.size());
    ever_used_.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) {
        // stack: the page given back last is handed out first, so pages are
        // used again as early as possible
        for (int p = groups_[g].num_pages - 1; p >= 0; --p) free_[g].push_back(p);
        ever_used_[g].assign(groups_[g].num_pages, 0);
    }
    for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
}

int CacheManager::admit(int64_t id) {
    if (reqs_.count(id)) return -2;
    if (free_slots_.empty()) return -1;
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.len = 0;
    r.blocks.resize(groups_.size());
    r.first_live.assign(groups_.size(), 0);
    reqs_.emplace(id, std::move(r));
    return reqs_[id].slot;
}

int CacheManager::first_needed_block(const Request& r, int g) const {
    // the next token sits at position r.len and reads positions > r.len - window
    const int w = groups_[g].window;
    if (w <= 0) return 0;
    const int first_pos = std::max(0, r.len - w + 1);
    return first_pos / groups_[g].page_size;
}

void CacheManager::trim(Request& r) {
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int keep_from = first_needed_block(r, (int)g);
        auto& b = r.blocks[g];
        for (int i = r.first_live[g]; i < keep_from && i < (int)b.size(); ++i) {
            if (b[i] >= 0) {
                free_[g].push_back(b[i]);
                b[i] = -1;
            }
        }
        r.first_live[g] = std::max(r.first_live[g], std::min(keep_from, (int)b.size()));
    }
}

int CacheManager::pages_needed(int64_t id, int n_new, int g) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -2;
    const Request& r = it->second;
    const int ps = groups_[g].page_size;
    const int blocks_after = (r.len + n_new + ps - 1) / ps;
    const int held = (int)r.blocks[g].size();
    int need = std::max(0, blocks_after - held);
    // pages that the window has passed come back before the new ones are taken
    int back = 0;
    const int keep_from = first_needed_block(r, g);
    for (int i = r.first_live[g]; i < keep_from && i < held; ++i)
        if (r.blocks[g][i] >= 0) ++back;
    return need - back;
}

int CacheManager::extend(int64_t id, int n_new) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -2;
    if (n_new < 0) return -3;
    Request& r = it->second;
    for (size_t g = 0; g < groups_.size(); ++g)
        if (pages_needed(id, n_new, (int)g) > (int)free_[g].size()) return -1;
    trim(r);
    for (size_t g = 0; g < groups_.size(); ++g) {
        const int ps = groups_[g].page_size;
        const int blocks_after = (r.len + n_new + ps - 1) / ps;
        auto& b = r.blocks[g];
        while ((int)b.size() < blocks_after) {
            const int32_t p = free_[g].back();
            free_[g].pop_back();
            if (ever_used_[g][p]) ++reused_;
            ever_used_[g][p] = 1;
            b.push_back(p);
        }
    }
    r.len += n_new;
    return 0;
}

int CacheManager::release(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -2;
    Request& r = it->second;
    for (size_t g = 0; g < groups_.size(); ++g)
        for (int32_t p : r.blocks[g])
            if (p >= 0) free_[g].push_back(p);
    free_slots_.push_back(r.slot);
    reqs_.erase(it);
    return 0;
}

int CacheManager::length(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -2 : it->second.len;
}

int CacheManager::slot(int64_t id) const {
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -2 : it->second.slot;
}

int CacheManager::block_table(int64_t id, int g, int32_t* out, int capacity) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -2;
    const auto& b = it->second.blocks[g];
    const int n = std::min((int)b.size(), capacity);
    for (int i = 0; i < n; ++i) out[i] = b[i];
    for (int i = n; i < capacity; ++i) out[i] = -1;
    return (int)b.size();
}

int CacheManager::fill_step(int n, const int64_t* ids, const int32_t* counts, int32_t* meta,
                            int off_positions, int off_tok_entry, int off_cu_q, int off_kv_len,
                            int off_slots, const int32_t* off_tables, const int32_t* max_blocks) const {
    int row = 0;
    meta[off_cu_q] = 0;
    for (int i = 0; i < n; ++i) {
        auto it = reqs_.find(ids[i]);
        if (it == reqs_.end()) return -2;
        const Request& r = it->second;
        const int c = counts[i], start = r.len - c;
        for (int t = 0; t < c; ++t) {
            meta[off_positions + row + t] = start + t;
            meta[off_tok_entry + row + t] = i;
        }
        row += c;
        meta[off_cu_q + i + 1] = row;
        meta[off_kv_len + i] = r.len;
        meta[off_slots + i] = r.slot;
        for (size_t g = 0; g < groups_.size(); ++g) {
            int32_t* out = meta + off_tables[g] + (long long)i * max_blocks[g];
            const auto& b = r.blocks[g];
            const int m = std::min((int)b.size(), (int)max_blocks[g]);
            for (int k = 0; k < m; ++k) out[k] = b[k];
            for (int k = m; k < max_blocks[g]; ++k) out[k] = -1;
        }
    }
    return row;
}

int CacheManager::check() const {
    std::vector<int> slot_seen(max_requests_, 0);
    for (int s : free_slots_) {
        if (s < 0 || s >= max_requests_ || slot_seen[s]++) return 1;
    }
    for (const auto& kv : reqs_) {
        const int s = kv.second.slot;
        if (s < 0 || s >= max_requests_ || slot_seen[s]++) return 2;
    }
    for (int s = 0; s < max_requests_; ++s)
        if (slot_seen[s] != 1) return 3;
    for (size_t g = 0; g < groups_.size(); ++g) {
        std::vector<int> seen(groups_[g].num_pages, 0);
        for (int32_t p : free_[g]) {
            if (p < 0 || p >= groups_[g].num_pages || seen[p]++) return 4;
        }
        for (const auto& kv : reqs_)
            for (int32_t p : kv.second.blocks[g]) {
                if (p < 0) continue;
                if (p >= groups_[g].num_pages || seen[p]++) return 5;
            }
        for (int p = 0; p < groups_[g].num_pages; ++p)
            if (seen[p] != 1) return 6;   // a page was lost
    }
    return 0;
}

}  // namespace crane

using crane::CacheManager;

CRANE_HOST_API void* crane_cache_create(int n_groups, const int* num_pages, const int* page_size,
                                        const int* window, int max_requests) {
    std::vector<crane::GroupSpec> g;
    for (int i = 0; i < n_groups; ++i) {
        if (num_pages[i] < 0 || page_size[i] <= 0 || window[i] < 0) return nullptr;
        g.push_back({num_pages[i], page_size[i], window[i]});
    }
    if (max_requests <= 0) return nullptr;
    return new CacheManager(g, max_requests);
}
CRANE_HOST_API void crane_cache_destroy(void* c) { delete (CacheManager*)c; }
CRANE_HOST_API int crane_cache_admit(void* c, int64_t id) { return ((CacheManager*)c)->admit(id); }
CRANE_HOST_API int crane_cache_extend(void* c, int64_t id, int n) {
    return ((CacheManager*)c)->extend(id, n);
}
CRANE_HOST_API int crane_cache_pages_needed(void* c, int64_t id, int n, int g) {
    return ((CacheManager*)c)->pages_needed(id, n, g);
}
CRANE_HOST_API int crane_cache_release(void* c, int64_t id) {
    return ((CacheManager*)c)->release(id);
}
CRANE_HOST_API int crane_cache_length(void* c, int64_t id) { return ((CacheManager*)c)->length(id); }
CRANE_HOST_API int crane_cache_slot(void* c, int64_t id) { return ((CacheManager*)c)->slot(id); }
CRANE_HOST_API int crane_cache_block_table(void* c, int64_t id, int g, int32_t* out, int cap) {
    return ((CacheManager*)c)->block_table(id, g, out, cap);
}
CRANE_HOST_API int crane_cache_fill_step(void* c, int n, const int64_t* ids, const int32_t* counts,
                                         int32_t* meta, int off_positions, int off_tok_entry,
                                         int off_cu_q, int off_kv_len, int off_slots,
                                         const int32_t* off_tables, const int32_t* max_blocks) {
    return ((CacheManager*)c)->fill_step(n, ids, counts, meta, off_positions, off_tok_entry, off_cu_q,
                                         off_kv_len, off_slots, off_tables, max_blocks);
}
CRANE_HOST_API int crane_cache_free_pages(void* c, int g) {
    return ((CacheManager*)c)->free_pages(g);
}
CRANE_HOST_API int crane_cache_total_pages(void* c, int g) {
    return ((CacheManager*)c)->total_pages(g);
}
CRANE_HOST_API int crane_cache_free_slots(void* c) { return ((CacheManager*)c)->free_slots(); }
CRANE_HOST_API int crane_cache_live(void* c) { return ((CacheManager*)c)->live_requests(); }
CRANE_HOST_API int64_t crane_cache_pages_reused(void* c) {
    return ((CacheManager*)c)->pages_reused();
}
CRANE_HOST_API int crane_cache_check(void* c) { return ((CacheManager*)c)->check(); }
