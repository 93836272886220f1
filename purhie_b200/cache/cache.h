// The cache manager: paged keys and values with a block table per request, and state slots.
//
// Each entry of a model's run order tells the manager what it needs (CacheNeed): pages holding all keys, pages
// holding a window of them, a fixed-size state per request, or nothing.  Entries with the same page geometry
// and the same policy form a group; a group has a pool of pages of its own, one page id addresses the keys and
// values of all the group's entries (the reference's "one block, all layers" layout, src/kv_cache.h:1-14), and
// every live request has one block table per group.  Pages go back to the pool when a request is released and,
// in a window group, as soon as the window has passed them (the reference keeps window layers in a second,
// ring-shaped cache: src/inference.cpp:1594-1609, 1650-1665).  Beside the pages there are max_requests state
// slots (the reference's per-sequence RecurrentState, src/qwen_model.cpp:319-391, 620-634), zeroed when a request
// is admitted.  The reference itself keeps one cache per sequence, made of blocks of 256 positions that are never
// given back before the sequence is freed (src/kv_cache.cpp:133-226, 242-260; src/inference.cpp:1784-1802).
//
// A page of a group is laid out [entry][K|V][kv_head][token in page][head_dim] (the V part value_dim wide where a
// mixer's values are not as wide as its keys).
// The bookkeeping touches no device until materialize(), so it is tested without one.
#pragma once

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../host/common.h"
#include "../host/device.h"
#include "../parts/parts.h"

namespace qe {

// num_pages pages numbered from 0.  A page is free or held with a reference count >= 1 (the counts are kept for
// sharing a page between requests; the reference shares blocks with a store, src/kv_cache.cpp:266-347).
class QE_API PageAllocator {
public:
    explicit PageAllocator(int num_pages = 0);
    int num_pages() const { return (int)ref_.size(); }
    int num_free() const { return (int)free_.size(); }
    std::vector<int> alloc(int n);                 // OutOfPages, taking nothing, when fewer than n are free
    void share(int page);
    int refcount(int page) const { return ref_.at(page); }
    std::vector<int> free(const std::vector<int>& pages);   // drops one reference each; returns the pages now free
    void check() const;
private:
    std::vector<int> free_;                        // a stack: the page freed last is handed out first
    std::vector<int> ref_;
};

class QE_API SlotAllocator {
public:
    explicit SlotAllocator(int num_slots = 0);
    int num_slots() const { return (int)held_.size(); }
    int num_free() const { return (int)free_.size(); }
    int alloc();                                   // OutOfSlots when all are in use
    void free(int slot);
    void check() const;
private:
    std::vector<int> free_;
    std::vector<char> held_;
};

struct PageGroup {
    int index = 0;
    int kv_heads = 0, head_dim = 0, value_dim = 0, window = 0;      // value_dim: as CacheNeed::v_dim()
    std::vector<int> entries;                      // run-order entries whose keys and values live in this group
    PageAllocator allocator;
    // [entries, pages, {K: kv_heads x page_size x head_dim, V: ... x value_dim}]: what one layer's attention reads lies
    // together (a pool of tens of GB with the layers interleaved page by page spreads every layer over all of it,
    // and the address translations of a layer's pages stop fitting the translation caches)
    DeviceBuffer pool;
    long long page_stride = 0;                     // elements of one entry's page (keys and values)
    int entry_slot(int entry) const;
};

struct RequestCache {
    int64_t id = 0;
    int length = 0;                                // tokens whose keys are in the cache
    std::vector<std::vector<int>> tables;          // per group: page of each logical block, -1 once freed
    std::vector<int> first_live;                   // per group: first logical block still held
    int slot = -1;
};

class QE_API CacheManager {
public:
    // needs[i] is the need of run-order entry i (an entry that borrows another entry's cache has kind None).
    // num_pages: one number for every group, or one per group in the order in which groups first appear.
    CacheManager(std::vector<CacheNeed> needs, int page_size, std::vector<int> num_pages, int max_requests);

    // Allocate the pools and the state on the current device.  poison fills pages with NaN at the start and
    // whenever they are freed, so that a kernel that reads a position it must not see shows.
    void materialize(DType dtype, bool poison, cudaStream_t stream);
    size_t pool_bytes() const;

    // ---- requests
    void add_request(int64_t id);                  // OutOfSlots; zeroes the request's state
    bool has_request(int64_t id) const { return requests_.count(id) != 0; }
    int length(int64_t id) const { return get(id).length; }
    std::vector<int> pages_needed(int64_t id, int n_new) const;        // what reserve() would take from each group
    std::vector<int> pages_for_new_request(int n_tokens) const;
    std::vector<int> free_pages() const;
    std::vector<int> total_pages() const;
    bool can_reserve(int64_t id, int n_new) const;
    void reserve(int64_t id, int n_new);           // pages for positions [length, length + n_new) in every group, or OutOfPages and nothing
    void unreserve(int64_t id);                    // give back the pages reserved beyond the request's length
    void advance(int64_t id, int n_new);           // the tokens are in the cache now; window groups give back what no later position sees
    void truncate(int64_t id, int length);         // forget everything from `length` on; not with windows or state
    bool can_rewind() const;                       // no window group and no state entry
    void release(int64_t id);

    // ---- what a step needs
    const std::vector<int>& block_table(int64_t id, int group) const { return get(id).tables.at(group); }
    int slot_of(int64_t id) const { return get(id).slot; }
    void token_slots(int64_t id, int group, int start, int n, std::vector<int32_t>& out) const;   // appends page * page_size + offset
    CacheView view(int entry, int owner) const;    // the cache of run-order entry `owner` as entry `entry` sees it

    void check() const;                            // CheckError unless no page is lost, held twice or free while held

    int page_size() const { return page_size_; }
    int max_requests() const { return max_requests_; }
    const std::vector<CacheNeed>& needs() const { return needs_; }
    const std::vector<PageGroup>& groups() const { return groups_; }
    int entry_group(int entry) const;              // -1 when the entry has no pages
    const std::vector<int>& state_entries() const { return state_entries_; }
    const SlotAllocator& slots() const { return slots_; }
    const std::unordered_map<int64_t, RequestCache>& requests() const { return requests_; }
    DType dtype() const { return dtype_; }

private:
    const RequestCache& get(int64_t id) const;
    RequestCache& get(int64_t id);
    int first_needed_block(const PageGroup& g, int start) const;
    void free_pages_of(PageGroup& g, const std::vector<int>& pages);

    int page_size_, max_requests_;
    std::vector<CacheNeed> needs_;
    std::vector<PageGroup> groups_;
    std::map<int, int> entry_group_;
    std::vector<int> state_entries_;
    SlotAllocator slots_;
    std::map<int, DeviceBuffer> state_;            // entry -> [max_requests, *state_shape]
    std::unordered_map<int64_t, RequestCache> requests_;
    DType dtype_ = DType::F32;
    bool poison_ = false, materialized_ = false;
    cudaStream_t stream_ = nullptr;
};

}  // namespace qe
