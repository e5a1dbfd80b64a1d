// Page pool: free list + reference counts for the paged KV cache, and a first-fit range
// heap (256-byte alignment, coalescing free list) for arena sub-allocation.
//
// Reference behaviour: page refcounts in `src/paged_kv.ts:25-531`; `Heap` in
// `src/heap.ts:1-209`.  Plain C ABI so that Python (ctypes) and C++ callers share it.
#include <algorithm>
#include <cstdint>
#include <map>
#include <mutex>
#include <vector>

#define RT_API extern "C" __attribute__((visibility("default")))

namespace {

struct PagePool {
    std::vector<int32_t> refs;
    std::vector<int32_t> free_list;     // LIFO: recently freed pages are reused first
    std::mutex mu;
    explicit PagePool(int n) : refs(n, 0) {
        free_list.reserve(n);
        for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
    }
};

struct Heap {
    uint64_t capacity, alignment, used = 0;
    std::map<uint64_t, uint64_t> free_by_offset;   // offset -> size
    std::map<uint64_t, uint64_t> live;             // offset -> size
    std::mutex mu;
    Heap(uint64_t cap, uint64_t align) : capacity(cap), alignment(align) { free_by_offset[0] = cap; }
};

}  // namespace

RT_API void* rt_pool_create(int num_pages) { return new PagePool(num_pages); }
RT_API void rt_pool_destroy(void* p) { delete static_cast<PagePool*>(p); }
RT_API int rt_pool_free_count(void* p) {
    auto* pool = static_cast<PagePool*>(p);
    std::lock_guard<std::mutex> g(pool->mu);
    return (int)pool->free_list.size();
}
// Allocates n pages (refcount 1 each) into out[]; returns 0, or -1 (nothing allocated) if fewer are free.
RT_API int rt_pool_alloc(void* p, int n, int32_t* out) {
    auto* pool = static_cast<PagePool*>(p);
    std::lock_guard<std::mutex> g(pool->mu);
    if ((int)pool->free_list.size() < n) return -1;
    for (int i = 0; i < n; ++i) {
        const int32_t id = pool->free_list.back();
        pool->free_list.pop_back();
        pool->refs[id] = 1;
        out[i] = id;
    }
    return 0;
}
RT_API int rt_pool_ref(void* p, int page) {
    auto* pool = static_cast<PagePool*>(p);
    std::lock_guard<std::mutex> g(pool->mu);
    if (page < 0 || page >= (int)pool->refs.size() || pool->refs[page] <= 0) return -1;
    return ++pool->refs[page];
}
RT_API int rt_pool_unref(void* p, int page) {
    auto* pool = static_cast<PagePool*>(p);
    std::lock_guard<std::mutex> g(pool->mu);
    if (page < 0 || page >= (int)pool->refs.size() || pool->refs[page] <= 0) return -1;
    if (--pool->refs[page] == 0) pool->free_list.push_back(page);
    return pool->refs[page];
}
RT_API int rt_pool_refcount(void* p, int page) {
    auto* pool = static_cast<PagePool*>(p);
    std::lock_guard<std::mutex> g(pool->mu);
    if (page < 0 || page >= (int)pool->refs.size()) return -1;
    return pool->refs[page];
}

// Longest common prefix of two token arrays (prefix-cache scan).
RT_API int64_t rt_common_prefix(const int64_t* a, int64_t na, const int64_t* b, int64_t nb) {
    const int64_t n = std::min(na, nb);
    int64_t i = 0;
    while (i < n && a[i] == b[i]) ++i;
    return i;
}

// ---- heap -------------------------------------------------------------------------------------------
RT_API void* rt_heap_create(uint64_t capacity, uint64_t alignment) { return new Heap(capacity, alignment ? alignment : 256); }
RT_API void rt_heap_destroy(void* h) { delete static_cast<Heap*>(h); }
// First fit.  Returns the offset or UINT64_MAX.
RT_API uint64_t rt_heap_alloc(void* hp, uint64_t size) {
    auto* h = static_cast<Heap*>(hp);
    std::lock_guard<std::mutex> g(h->mu);
    if (size == 0) size = 1;
    size = (size + h->alignment - 1) / h->alignment * h->alignment;
    for (auto it = h->free_by_offset.begin(); it != h->free_by_offset.end(); ++it) {
        if (it->second >= size) {
            const uint64_t off = it->first, rest = it->second - size;
            h->free_by_offset.erase(it);
            if (rest) h->free_by_offset[off + size] = rest;
            h->live[off] = size;
            h->used += size;
            return off;
        }
    }
    return UINT64_MAX;
}
RT_API int rt_heap_free(void* hp, uint64_t offset) {
    auto* h = static_cast<Heap*>(hp);
    std::lock_guard<std::mutex> g(h->mu);
    auto it = h->live.find(offset);
    if (it == h->live.end()) return -1;
    uint64_t off = it->first, size = it->second;
    h->live.erase(it);
    h->used -= size;
    auto next = h->free_by_offset.lower_bound(off);
    if (next != h->free_by_offset.end() && off + size == next->first) {
        size += next->second;
        next = h->free_by_offset.erase(next);
    }
    if (next != h->free_by_offset.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) {
            prev->second += size;
            return 0;
        }
    }
    h->free_by_offset[off] = size;
    return 0;
}
RT_API uint64_t rt_heap_used(void* hp) { return static_cast<Heap*>(hp)->used; }
RT_API uint64_t rt_heap_largest_free(void* hp) {
    auto* h = static_cast<Heap*>(hp);
    std::lock_guard<std::mutex> g(h->mu);
    uint64_t best = 0;
    for (auto& kv : h->free_by_offset) best = std::max(best, kv.second);
    return best;
}
RT_API int rt_heap_num_free_ranges(void* hp) { return (int)static_cast<Heap*>(hp)->free_by_offset.size(); }
