// Host-side bookkeeping of the paged key/value cache and of the per-request
// state slots.  No device memory is touched here: the manager deals in page
// numbers and slot numbers; the tensors they index belong to the engine.
//
// Layers with the same cache need form a group.  Every group has its own pool
// of pages, its own page size and, per request, its own block table (logical
// block -> physical page, -1 where no page is held).  A group with window W > 0
// only ever needs the last W positions; its pages are given back as soon as
// every position on them has fallen out of the window of the next token.
//
// The reference keeps one contiguous cache tensor per sequence and swaps whole
// tensors in and out of the model
// (crane-core/src/models/hunyuan_dense/modeling.rs:433-489,
// crane-serve/src/engine/mod.rs:1214-1271); pages replace both.
#pragma once
#include <cstdint>
#include <unordered_map>
#include <vector>

namespace crane {

struct GroupSpec {
    int num_pages;
    int page_size;
    int window;   // 0: every earlier position stays readable
};

class CacheManager {
public:
    CacheManager(const std::vector<GroupSpec>& groups, int max_requests);

    // A state slot for a new request; -1 if none is free, -2 if the id is live.
    int admit(int64_t id);
    // Pages for `n_new` more tokens of a live request, all groups or none:
    // 0 on success; -1 if some group lacks pages (nothing changes); -2 unknown id.
    int extend(int64_t id, int n_new);
    // How many pages extend(id, n_new) would take from group g (after giving
    // back what the window has passed); -2 unknown id.
    int pages_needed(int64_t id, int n_new, int g) const;
    // Give back everything the request holds.  0, or -2 for an unknown id.
    int release(int64_t id);

    int length(int64_t id) const;       // tokens cached, -2 unknown
    int slot(int64_t id) const;         // state slot, -2 unknown
    // Copies the request's block table of group g; entries beyond the held
    // blocks are -1.  Returns the number of logical blocks in use, -2 unknown.
    int block_table(int64_t id, int g, int32_t* out, int capacity) const;

    // Lays out the metadata of one step for `n` live requests whose pages are
    // already taken: entry i has `counts[i]` new tokens, the last of which sits
    // at position length(ids[i]) - 1.  Writes into `meta` at the given offsets
    // (in int32 units): positions and tok_entry per token, cu_q [n + 1], kv_len
    // and slots per entry, and per group the block-table rows [n][max_blocks[g]].
    // Returns the number of tokens, or -2 for an unknown id.
    int fill_step(int n, const int64_t* ids, const int32_t* counts, int32_t* meta, int off_positions,
                  int off_tok_entry, int off_cu_q, int off_kv_len, int off_slots,
                  const int32_t* off_tables, const int32_t* max_blocks) const;

    int num_groups() const { return (int)groups_.size(); }
    int free_pages(int g) const { return (int)free_[g].size(); }
    int total_pages(int g) const { return groups_[g].num_pages; }
    int page_size(int g) const { return groups_[g].page_size; }
    int free_slots() const { return (int)free_slots_.size(); }
    int live_requests() const { return (int)reqs_.size(); }
    int64_t pages_reused() const { return reused_; }
    // 0 if every page and slot is either free or held by exactly one request.
    int check() const;

private:
    struct Request {
        int slot;
        int len;
        std::vector<std::vector<int32_t>> blocks;   // per group: physical page or -1
        std::vector<int> first_live;                 // per group: first block still held
    };
    void trim(Request& r);
    int first_needed_block(const Request& r, int g) const;

    std::vector<GroupSpec> groups_;
    std::vector<std::vector<int32_t>> free_;   // per group, used as a stack
    std::vector<std::vector<uint8_t>> ever_used_;
    std::vector<int> free_slots_;
    std::unordered_map<int64_t, Request> reqs_;
    int max_requests_;
    int64_t reused_ = 0;
};

}  // namespace crane
