#include "cache.h"

#include <algorithm>
#include <set>

namespace qe {

// ---- pages and slots -------------------------------------------------------------------------------------------
PageAllocator::PageAllocator(int num_pages) {
    if (num_pages < 0) throw Error(kInvalidArg, "num_pages must be >= 0");
    ref_.assign(num_pages, 0);
    free_.reserve(num_pages);
    for (int p = num_pages - 1; p >= 0; p--) free_.push_back(p);
}
std::vector<int> PageAllocator::alloc(int n) {
    if (n < 0) throw Error(kInvalidArg, "cannot allocate a negative number of pages");
    if (n > (int)free_.size())
        throw OutOfPages(std::to_string(n) + " pages wanted, " + std::to_string(free_.size()) + " of " + std::to_string(ref_.size()) + " free");
    std::vector<int> pages;
    pages.reserve(n);
    for (int i = 0; i < n; i++) {
        pages.push_back(free_.back());
        free_.pop_back();
        ref_[pages.back()] = 1;
    }
    return pages;
}
void PageAllocator::share(int page) {
    if (page < 0 || page >= (int)ref_.size() || ref_[page] < 1)
        throw Error(kInvalidArg, "page " + std::to_string(page) + " is free and cannot be shared");
    ref_[page]++;
}
std::vector<int> PageAllocator::free(const std::vector<int>& pages) {
    std::vector<int> released;
    for (int p : pages) {
        if (p < 0 || p >= (int)ref_.size()) throw CheckError("page " + std::to_string(p) + " is outside the pool of " + std::to_string(ref_.size()));
        if (ref_[p] < 1) throw CheckError("page " + std::to_string(p) + " freed twice");
        if (--ref_[p] == 0) {
            free_.push_back(p);
            released.push_back(p);
        }
    }
    return released;
}
void PageAllocator::check() const {
    std::set<int> free(free_.begin(), free_.end());
    if (free.size() != free_.size()) throw CheckError("a page is on the free list twice");
    for (int p = 0; p < (int)ref_.size(); p++)
        if ((ref_[p] == 0) != (free.count(p) != 0))
            throw CheckError("page " + std::to_string(p) + ": refcount " + std::to_string(ref_[p]) + ", on free list: " +
                             (free.count(p) ? "yes" : "no"));
}

SlotAllocator::SlotAllocator(int num_slots) {
    held_.assign(std::max(num_slots, 0), 0);
    for (int s = num_slots - 1; s >= 0; s--) free_.push_back(s);
}
int SlotAllocator::alloc() {
    if (free_.empty()) throw OutOfSlots("all " + std::to_string(held_.size()) + " state slots are in use");
    int s = free_.back();
    free_.pop_back();
    held_[s] = 1;
    return s;
}
void SlotAllocator::free(int slot) {
    if (slot < 0 || slot >= (int)held_.size() || !held_[slot]) throw CheckError("slot " + std::to_string(slot) + " is not held");
    held_[slot] = 0;
    free_.push_back(slot);
}
void SlotAllocator::check() const {
    std::set<int> free(free_.begin(), free_.end());
    if (free.size() != free_.size()) throw CheckError("a slot is on the free list twice");
    for (int s = 0; s < (int)held_.size(); s++)
        if ((held_[s] != 0) == (free.count(s) != 0)) throw CheckError("slot " + std::to_string(s) + " is both held and free, or neither");
}

int PageGroup::entry_slot(int entry) const {
    for (size_t i = 0; i < entries.size(); i++) if (entries[i] == entry) return (int)i;
    throw Error(kInvalidState, "entry " + std::to_string(entry) + " is not in this page group");
}

// ---- the manager ---------------------------------------------------------------------------------------------------
CacheManager::CacheManager(std::vector<CacheNeed> needs, int page_size, std::vector<int> num_pages, int max_requests)
    : page_size_(page_size), max_requests_(max_requests), needs_(std::move(needs)), slots_(max_requests) {
    if (page_size < 1) throw Error(kInvalidArg, "page_size must be >= 1");
    if (max_requests < 1) throw Error(kInvalidArg, "max_requests must be >= 1");
    for (int i = 0; i < (int)needs_.size(); i++) {
        const CacheNeed& need = needs_[i];
        if (need.kind == CacheNeed::State) state_entries_.push_back(i);
        if (need.kind != CacheNeed::Pages) continue;
        int gi = -1;
        for (const PageGroup& g : groups_)
            if (g.kv_heads == need.kv_heads && g.head_dim == need.head_dim && g.value_dim == need.v_dim() && g.window == need.window) gi = g.index;
        if (gi < 0) {
            PageGroup g;
            g.index = gi = (int)groups_.size();
            g.kv_heads = need.kv_heads; g.head_dim = need.head_dim; g.value_dim = need.v_dim(); g.window = need.window;
            groups_.push_back(std::move(g));
        }
        groups_[gi].entries.push_back(i);
        entry_group_[i] = gi;
    }
    if (num_pages.size() == 1 && groups_.size() != 1) num_pages.assign(groups_.size(), num_pages[0]);
    if (num_pages.size() != groups_.size())
        throw Error(kInvalidArg, std::to_string(num_pages.size()) + " page counts for " + std::to_string(groups_.size()) + " groups");
    for (size_t i = 0; i < groups_.size(); i++) {
        groups_[i].allocator = PageAllocator(num_pages[i]);
        // one entry's keys and values of one page; an entry's pages lie side by side, the entries one after the other
        groups_[i].page_stride = (long long)groups_[i].kv_heads * page_size_ * (groups_[i].head_dim + groups_[i].value_dim);
    }
}

void CacheManager::materialize(DType dtype, bool poison, cudaStream_t stream) {
    dtype_ = dtype; poison_ = poison; stream_ = stream;
    for (PageGroup& g : groups_) {
        size_t bytes = g.entries.size() * (size_t)g.allocator.num_pages() * (size_t)g.page_stride * dtype_size(dtype);
        g.pool = DeviceBuffer(std::max<size_t>(bytes, 16));
        // all bits set is a NaN in float32 and in bfloat16
        QE_CUDA(cudaMemsetAsync(g.pool.data(), poison ? 0xFF : 0, g.pool.bytes(), stream));
    }
    for (int e : state_entries_) {
        Tensor t(nullptr, needs_[e].state_dtype, needs_[e].state_shape);
        size_t bytes = (size_t)max_requests_ * t.bytes();
        state_[e] = DeviceBuffer(std::max<size_t>(bytes, 16));
        QE_CUDA(cudaMemsetAsync(state_[e].data(), 0, state_[e].bytes(), stream));
    }
    QE_CUDA(cudaStreamSynchronize(stream));
    materialized_ = true;
}

size_t CacheManager::pool_bytes() const {
    size_t n = 0;
    for (const PageGroup& g : groups_) n += g.pool.bytes();
    return n;
}

const RequestCache& CacheManager::get(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw Error(kInvalidArg, "request " + std::to_string(id) + " is not live");
    return it->second;
}
RequestCache& CacheManager::get(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw Error(kInvalidArg, "request " + std::to_string(id) + " is not live");
    return it->second;
}

void CacheManager::add_request(int64_t id) {
    if (requests_.count(id)) throw Error(kInvalidArg, "request " + std::to_string(id) + " is already live");
    RequestCache rc;
    rc.id = id;
    rc.slot = slots_.alloc();
    rc.tables.assign(groups_.size(), {});
    rc.first_live.assign(groups_.size(), 0);
    if (materialized_)
        for (int e : state_entries_) {
            Tensor t(nullptr, needs_[e].state_dtype, needs_[e].state_shape);
            QE_CUDA(cudaMemsetAsync(static_cast<char*>(state_[e].data()) + (size_t)rc.slot * t.bytes(), 0, t.bytes(), stream_));
        }
    requests_.emplace(id, std::move(rc));
}

int CacheManager::first_needed_block(const PageGroup& g, int start) const {
    if (!g.window) return 0;
    return std::max(0, start - g.window + 1) / page_size_;
}

std::vector<int> CacheManager::pages_needed(int64_t id, int n_new) const {
    const RequestCache& rc = get(id);
    const int blocks = (rc.length + n_new + page_size_ - 1) / page_size_;
    std::vector<int> out;
    for (const PageGroup& g : groups_) out.push_back(std::max(0, blocks - (int)rc.tables[g.index].size()));
    return out;
}
std::vector<int> CacheManager::pages_for_new_request(int n_tokens) const {
    return std::vector<int>(groups_.size(), (n_tokens + page_size_ - 1) / page_size_);
}
std::vector<int> CacheManager::free_pages() const {
    std::vector<int> out;
    for (const PageGroup& g : groups_) out.push_back(g.allocator.num_free());
    return out;
}
std::vector<int> CacheManager::total_pages() const {
    std::vector<int> out;
    for (const PageGroup& g : groups_) out.push_back(g.allocator.num_pages());
    return out;
}
bool CacheManager::can_reserve(int64_t id, int n_new) const {
    std::vector<int> need = pages_needed(id, n_new);
    for (size_t i = 0; i < groups_.size(); i++) if (need[i] > groups_[i].allocator.num_free()) return false;
    return true;
}

void CacheManager::reserve(int64_t id, int n_new) {
    RequestCache& rc = get(id);
    std::vector<int> need = pages_needed(id, n_new);
    for (size_t i = 0; i < groups_.size(); i++)
        if (need[i] > groups_[i].allocator.num_free())
            throw OutOfPages("request " + std::to_string(id) + ": group " + std::to_string(i) + " needs " + std::to_string(need[i]) +
                             " pages for " + std::to_string(n_new) + " more tokens, " + std::to_string(groups_[i].allocator.num_free()) +
                             " of " + std::to_string(groups_[i].allocator.num_pages()) + " free");
    for (size_t i = 0; i < groups_.size(); i++) {
        std::vector<int> pages = groups_[i].allocator.alloc(need[i]);
        rc.tables[i].insert(rc.tables[i].end(), pages.begin(), pages.end());
    }
}

void CacheManager::unreserve(int64_t id) {
    RequestCache& rc = get(id);
    const int blocks = (rc.length + page_size_ - 1) / page_size_;
    for (PageGroup& g : groups_) {
        std::vector<int>& table = rc.tables[g.index];
        if ((int)table.size() <= blocks) continue;
        std::vector<int> back;
        for (size_t b = blocks; b < table.size(); b++) if (table[b] >= 0) back.push_back(table[b]);
        free_pages_of(g, back);
        table.resize(blocks);
    }
}

void CacheManager::advance(int64_t id, int n_new) {
    RequestCache& rc = get(id);
    rc.length += n_new;
    if (!groups_.empty() && rc.length > (int)rc.tables[0].size() * page_size_)
        throw Error(kInvalidState, "request " + std::to_string(id) + " advanced past its reserved pages");
    for (PageGroup& g : groups_) {
        if (!g.window) continue;
        std::vector<int>& table = rc.tables[g.index];
        const int keep_from = std::min(first_needed_block(g, rc.length), (int)table.size());
        std::vector<int> passed;
        for (int b = rc.first_live[g.index]; b < keep_from; b++) {
            if (table[b] >= 0) passed.push_back(table[b]);
            table[b] = -1;
        }
        if (!passed.empty()) free_pages_of(g, passed);
        rc.first_live[g.index] = std::max(rc.first_live[g.index], keep_from);
    }
}

bool CacheManager::can_rewind() const {
    for (const PageGroup& g : groups_) if (g.window) return false;
    return state_entries_.empty();
}

void CacheManager::truncate(int64_t id, int length) {
    RequestCache& rc = get(id);
    if (length > rc.length || length < 0) throw Error(kInvalidArg, "truncate cannot lengthen a request");
    if (!can_rewind() && length != rc.length) throw Error(kInvalidState, "a request with windowed pages or state cannot be rewound");
    const int blocks = (length + page_size_ - 1) / page_size_;
    for (PageGroup& g : groups_) {
        std::vector<int>& table = rc.tables[g.index];
        if ((int)table.size() <= blocks) continue;
        std::vector<int> back;
        for (size_t b = blocks; b < table.size(); b++) if (table[b] >= 0) back.push_back(table[b]);
        free_pages_of(g, back);
        table.resize(blocks);
    }
    rc.length = length;
}

void CacheManager::release(int64_t id) {
    RequestCache& rc = get(id);
    for (PageGroup& g : groups_) {
        std::vector<int> back;
        for (int p : rc.tables[g.index]) if (p >= 0) back.push_back(p);
        free_pages_of(g, back);
    }
    slots_.free(rc.slot);
    requests_.erase(id);
}

void CacheManager::free_pages_of(PageGroup& g, const std::vector<int>& pages) {
    std::vector<int> released = g.allocator.free(pages);
    if (poison_ && materialized_) {
        // the page of every entry of the group: rows of a 2-D fill, one entry's region apart
        const size_t bytes = (size_t)g.page_stride * dtype_size(dtype_);
        const size_t entry_bytes = (size_t)g.allocator.num_pages() * bytes;
        for (int p : released)
            QE_CUDA(cudaMemset2DAsync(static_cast<char*>(g.pool.data()) + (size_t)p * bytes, entry_bytes, 0xFF, bytes, g.entries.size(), stream_));
    }
}

void CacheManager::token_slots(int64_t id, int group, int start, int n, std::vector<int32_t>& out) const {
    const std::vector<int>& table = get(id).tables.at(group);
    const int ps = page_size_;
    int p = start;
    while (p < start + n) {
        const int page = table.at(p / ps);
        if (page < 0) throw Error(kInvalidState, "request " + std::to_string(id) + ": position " + std::to_string(p) + " lies in a page that was given back");
        const int stop = std::min(start + n, (p / ps + 1) * ps);
        for (int q = p; q < stop; q++) out.push_back(page * ps + q % ps);
        p = stop;
    }
}

int CacheManager::entry_group(int entry) const {
    auto it = entry_group_.find(entry);
    return it == entry_group_.end() ? -1 : it->second;
}

CacheView CacheManager::view(int entry, int owner) const {
    CacheView v;
    const CacheNeed& need = needs_.at(owner);
    v.kind = need.kind;
    v.writable = (owner == entry);
    if (need.kind == CacheNeed::Pages) {
        const PageGroup& g = groups_[entry_group(owner)];
        const int slot = g.entry_slot(owner);
        const size_t elem = dtype_size(dtype_);
        const size_t k_elems = (size_t)g.kv_heads * page_size_ * g.head_dim;    // elements of the entry's keys in a page
        const size_t v_elems = (size_t)g.kv_heads * page_size_ * g.value_dim;   // ... and of its values
        char* base = static_cast<char*>(g.pool.data());
        v.group = g.index;
        const size_t entry_elems = (size_t)g.allocator.num_pages() * (k_elems + v_elems);   // all pages of one entry
        v.k_base = base + ((size_t)slot * entry_elems) * elem;
        v.v_base = base + ((size_t)slot * entry_elems + k_elems) * elem;
        v.kv_heads = g.kv_heads; v.key_dim = g.head_dim; v.value_dim = g.value_dim;
        v.kv_dtype = dtype_;
        v.page_stride = g.page_stride;
        v.page_size = page_size_;
        v.num_pages = g.allocator.num_pages();
    } else if (need.kind == CacheNeed::State) {
        std::vector<int64_t> shape = {max_requests_};
        shape.insert(shape.end(), need.state_shape.begin(), need.state_shape.end());
        auto it = state_.find(owner);
        v.state = Tensor(it == state_.end() ? nullptr : it->second.data(), need.state_dtype, shape);
    }
    return v;
}

void CacheManager::check() const {
    for (const PageGroup& g : groups_) {
        g.allocator.check();
        std::map<int, int> held;
        for (const auto& kv : requests_)
            for (int p : kv.second.tables[g.index]) if (p >= 0) held[p]++;
        for (int p = 0; p < g.allocator.num_pages(); p++) {
            const int h = held.count(p) ? held[p] : 0;
            if (g.allocator.refcount(p) != h)
                throw CheckError("group " + std::to_string(g.index) + " page " + std::to_string(p) + ": refcount " +
                                 std::to_string(g.allocator.refcount(p)) + ", held by " + std::to_string(h) + " tables");
        }
    }
    slots_.check();
    std::set<int> slots;
    for (const auto& kv : requests_) slots.insert(kv.second.slot);
    if (slots.size() != requests_.size()) throw CheckError("two requests share a state slot");
    if (slots_.num_free() != max_requests_ - (int)requests_.size()) throw CheckError("a state slot is lost");
}

}  // namespace qe
