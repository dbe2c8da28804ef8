// Free list of cache pages, host side, with a plain C interface.
//
// Same contract as the reference's BlockAllocator (include/firefly/scheduler.h:13-35,
// src/scheduler.cc:13-54): allocate(n) is all-or-nothing, free() gives pages back, and the
// list is last-in-first-out, so the page that was freed last is the next one handed out.
// On top of that every page's state is tracked: freeing a page twice, freeing a page the
// pool never gave out, and losing a page are detected and reported, not ignored.
// free() checks all ids before it changes anything.
#include <cstdint>
#include <vector>

namespace {

struct Pool {
    int num_blocks;
    int first_id;
    std::vector<int> free_list;      // back = next page handed out
    std::vector<uint8_t> held;       // 1: given out; 2: seen while checking
};

}  // namespace

#define FFH_EXPORT extern "C" __attribute__((visibility("default")))

FFH_EXPORT void* ffh_pool_create(int num_blocks, int first_id) {
    if (num_blocks < 0) return nullptr;
    Pool* p = new Pool{num_blocks, first_id, {}, std::vector<uint8_t>((size_t)num_blocks, 0)};
    p->free_list.reserve((size_t)num_blocks);
    for (int b = first_id + num_blocks - 1; b >= first_id; --b) p->free_list.push_back(b);   // lowest ids first
    return p;
}

FFH_EXPORT void ffh_pool_destroy(void* h) { delete static_cast<Pool*>(h); }

FFH_EXPORT int ffh_pool_num_free(void* h) { return (int)static_cast<Pool*>(h)->free_list.size(); }

// 1: n pages written to out; 0: fewer than n are free, nothing taken; -1: bad argument
FFH_EXPORT int ffh_pool_allocate(void* h, int n, int* out) {
    Pool* p = static_cast<Pool*>(h);
    if (n < 0) return -1;
    if ((size_t)n > p->free_list.size()) return 0;
    for (int i = 0; i < n; ++i) {
        const int b = p->free_list.back();
        p->free_list.pop_back();
        p->held[(size_t)(b - p->first_id)] = 1;
        out[i] = b;
    }
    return 1;
}

// 0: freed; 1: *bad_id does not belong to this pool; 2: *bad_id is not held (freed twice, or
// never allocated, or named twice in this call).  On 1 and 2 nothing has been changed.
FFH_EXPORT int ffh_pool_free(void* h, const int* ids, int n, int* bad_id) {
    Pool* p = static_cast<Pool*>(h);
    for (int i = 0; i < n; ++i) {
        const int idx = ids[i] - p->first_id;
        const bool foreign = idx < 0 || idx >= p->num_blocks;
        if (foreign || p->held[(size_t)idx] != 1) {
            *bad_id = ids[i];
            for (int j = 0; j < i; ++j) p->held[(size_t)(ids[j] - p->first_id)] = 1;   // undo the marks
            return foreign ? 1 : 2;
        }
        p->held[(size_t)idx] = 2;   // marks a second mention within this call
    }
    for (int i = 0; i < n; ++i) {
        p->held[(size_t)(ids[i] - p->first_id)] = 0;
        p->free_list.push_back(ids[i]);
    }
    return 0;
}

// 0: every page is free or held, exactly once; 1: *bad_id is on the free list twice; 2: *bad_id is
// both free and held; 3: a page was lost (neither free nor held).
FFH_EXPORT int ffh_pool_check(void* h, int* bad_id) {
    Pool* p = static_cast<Pool*>(h);
    std::vector<uint8_t> seen((size_t)p->num_blocks, 0);
    for (int b : p->free_list) {
        const size_t idx = (size_t)(b - p->first_id);
        if (seen[idx]) { *bad_id = b; return 1; }
        seen[idx] = 1;
        if (p->held[idx]) { *bad_id = b; return 2; }
    }
    size_t n_held = 0;
    for (uint8_t v : p->held) n_held += v != 0;
    if (p->free_list.size() + n_held != (size_t)p->num_blocks) { *bad_id = -1; return 3; }
    return 0;
}
