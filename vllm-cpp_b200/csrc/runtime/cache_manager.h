// Host side of the paged cache: page pools, per-request block tables, state slots.
//
// The reference keeps one pool whose pages cover every layer, allocates by a
// linear scan and rolls nothing back when a multi-page request fails half way
// (src/kv_cache_manager.cpp:43-54, 274-283).  Here layers are put in *groups* by
// what their mixer needs -- all keys of a request, or only a window of the last W
// keys -- and each group has a pool and a block table of its own.  Allocation is
// all-or-nothing over all groups, pages go back on a LIFO free list so a freed
// page is the next one handed out, and a window group gives pages back as soon as
// no later query can see them.  Beside the pages, every live request holds one
// *slot*: the index of its fixed-size per-request state on the device.
//
// Only integers live here; the device tensors that pages and slots index belong
// to the engine.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace vcb {

struct CacheError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// A LIFO pool of integer ids (pages or slots) that knows which ids are out.
class IdPool {
public:
    explicit IdPool(int32_t n);
    // Takes n ids or none; false when fewer than n are free.
    bool alloc(int32_t n, std::vector<int32_t>& out);
    // Gives one id back; throws on an id that is out of range or not held.
    void free(int32_t id);
    int32_t free_count() const { return (int32_t)free_.size(); }
    int32_t size() const { return (int32_t)held_.size(); }
    bool is_held(int32_t id) const { return id >= 0 && id < size() && held_[id]; }

private:
    std::vector<int32_t> free_;
    std::vector<uint8_t> held_;
};

struct GroupSpec {
    int32_t page_size = 16;  // tokens per page
    int32_t num_pages = 0;   // pages in this group's pool
    int32_t window = 0;      // 0: every key stays; W > 0: position p reads keys (p - W, p]
};

class CacheManager {
public:
    CacheManager(std::vector<GroupSpec> groups, int32_t num_slots);

    // Registers a request and takes its state slot.  Returns the slot, or -1 when all are taken.
    int32_t open(int64_t request);
    // Makes positions [0, new_len) addressable in every group.  All-or-nothing: on false nothing changed.
    bool reserve(int64_t request, int32_t new_len);
    // Records that new_len tokens are now cached; window groups give back pages every later query has passed.
    void commit(int64_t request, int32_t new_len);
    // Gives back the request's pages and slot.
    void close(int64_t request);

    bool is_open(int64_t request) const { return seqs_.count(request) != 0; }
    int32_t slot(int64_t request) const { return seq(request).slot; }
    int32_t num_tokens(int64_t request) const { return seq(request).committed; }
    int32_t reserved_tokens(int64_t request) const { return seq(request).reserved; }
    // Logical block -> page id of one group; -1 where a window has passed.
    const std::vector<int32_t>& block_table(int64_t request, int32_t group) const;

    int32_t num_groups() const { return (int32_t)groups_.size(); }
    const GroupSpec& group(int32_t g) const { return groups_.at(g); }
    int32_t free_pages(int32_t group) const { return pools_.at(group).free_count(); }
    int32_t free_slots() const { return slots_.free_count(); }
    int32_t num_open() const { return (int32_t)seqs_.size(); }

    // Pages group g must still hand out so that `request` (or a new one, request < 0) can reach new_len.
    int32_t pages_missing(int64_t request, int32_t group, int32_t new_len) const;
    // Largest number of pages of group g that one request of total_len tokens fed in portions of at
    // most `portion` tokens ever holds.
    int32_t peak_pages(int32_t group, int32_t total_len, int32_t portion) const;

    // Throws unless every page and slot is either free or held by exactly one request.
    void check_invariants() const;

private:
    struct Seq {
        int32_t slot = -1;
        int32_t committed = 0;
        int32_t reserved = 0;
        std::vector<std::vector<int32_t>> tables;  // [group][logical block]
    };
    const Seq& seq(int64_t request) const;
    Seq& seq(int64_t request);

    std::vector<GroupSpec> groups_;
    std::vector<IdPool> pools_;
    IdPool slots_;
    std::unordered_map<int64_t, Seq> seqs_;
};

}  // namespace vcb
