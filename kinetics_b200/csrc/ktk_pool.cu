// Host-side page pool for continuous batching: which physical pages of the paged KV cache belong
// to which sequence slot, handed out and taken back as sequences are admitted, grow and retire.
// No device code and no CUDA call: the pool only produces the CSR arrays (kv_indices, kv_indptr,
// kv_last_page_len) that the kernels read.
//
// The reference has no allocator: its benchmark builds one static interleaved table
// (benchmark/blocktopk_decoder.py:141) and its engine gives every slot max_seq_len tokens of cache
// up front (LiteSys/litesys/attention/batch_cache.py:32-40, engine.py:51-62).
#include <cstdint>
#include <new>
#include <cstring>
#include <vector>

#include "ktk_common.cuh"

struct ktk_pool {
    int64_t num_pages = 0;
    int32_t max_slots = 0;
    int32_t page_size = 0;
    std::vector<int32_t> free_list;              // stack: the page freed last is handed out first
    std::vector<std::vector<int32_t>> pages;     // per slot, in logical order
    std::vector<int64_t> tokens;                 // per slot, -1 = free slot
    std::vector<int64_t> reserved;               // per slot: pages promised at admission (>= pages held)
    int64_t promised = 0;                        // sum over slots of (reserved - held)
};

namespace {

inline int64_t pages_for(const ktk_pool* p, int64_t tokens) {
    return (tokens + p->page_size - 1) / p->page_size;
}

inline bool slot_ok(const ktk_pool* p, int32_t slot) { return p != nullptr && slot >= 0 && slot < p->max_slots; }

}  // namespace

using ktk::set_error;

extern "C" ktk_pool* ktk_pool_create(int64_t num_pages, int32_t max_slots, int32_t page_size) {
    if (num_pages <= 0 || num_pages > 2147483647LL || max_slots <= 0 || page_size <= 0) {
        set_error("ktk_pool_create: num_pages %lld, max_slots %d, page_size %d", (long long)num_pages, max_slots,
                  page_size);
        return nullptr;
    }
    ktk_pool* p = new (std::nothrow) ktk_pool;
    if (p == nullptr) {
        set_error("ktk_pool_create: out of host memory");
        return nullptr;
    }
    p->num_pages = num_pages;
    p->max_slots = max_slots;
    p->page_size = page_size;
    p->free_list.resize((size_t)num_pages);
    for (int64_t i = 0; i < num_pages; ++i) p->free_list[(size_t)i] = (int32_t)(num_pages - 1 - i);   // page 0 first
    p->pages.resize((size_t)max_slots);
    p->tokens.assign((size_t)max_slots, -1);
    p->reserved.assign((size_t)max_slots, 0);
    return p;
}

extern "C" void ktk_pool_destroy(ktk_pool* pool) { delete pool; }

extern "C" int64_t ktk_pool_free_pages(const ktk_pool* pool) {
    return pool ? (int64_t)pool->free_list.size() - pool->promised : -1;
}

extern "C" int64_t ktk_pool_slot_tokens(const ktk_pool* pool, int32_t slot) {
    return slot_ok(pool, slot) ? pool->tokens[(size_t)slot] : -1;
}

extern "C" int64_t ktk_pool_slot_pages(const ktk_pool* pool, int32_t slot) {
    return (slot_ok(pool, slot) && pool->tokens[(size_t)slot] >= 0) ? (int64_t)pool->pages[(size_t)slot].size() : -1;
}

extern "C" int ktk_pool_admit(ktk_pool* pool, int32_t slot, int64_t n_tokens, int64_t max_total_tokens) {
    if (!slot_ok(pool, slot) || n_tokens < 0 || max_total_tokens < n_tokens) {
        set_error("ktk_pool_admit: slot %d, %lld tokens now, %lld at most", slot, (long long)n_tokens,
                  (long long)max_total_tokens);
        return KTK_ERR_ARG;
    }
    if (pool->tokens[(size_t)slot] >= 0) {
        set_error("ktk_pool_admit: slot %d is in use", slot);
        return KTK_ERR_ARG;
    }
    const int64_t want = pages_for(pool, max_total_tokens);
    if (want > ktk_pool_free_pages(pool)) {
        set_error("ktk_pool_admit: %lld pages needed, %lld not promised to other sequences", (long long)want,
                  (long long)ktk_pool_free_pages(pool));
        return KTK_ERR_TOO_LARGE;
    }
    const int64_t now = pages_for(pool, n_tokens);
    std::vector<int32_t>& mine = pool->pages[(size_t)slot];
    mine.clear();
    for (int64_t i = 0; i < now; ++i) {
        mine.push_back(pool->free_list.back());
        pool->free_list.pop_back();
    }
    pool->tokens[(size_t)slot] = n_tokens;
    pool->reserved[(size_t)slot] = want;
    pool->promised += want - now;
    return KTK_OK;
}

extern "C" int ktk_pool_extend(ktk_pool* pool, const int32_t* slots, int32_t n, int32_t tokens_each) {
    if (pool == nullptr || (n > 0 && slots == nullptr) || n < 0 || tokens_each < 0) {
        set_error("ktk_pool_extend: bad arguments");
        return KTK_ERR_ARG;
    }
    // all or nothing: check first
    for (int32_t i = 0; i < n; ++i) {
        const int32_t s = slots[i];
        if (!slot_ok(pool, s) || pool->tokens[(size_t)s] < 0) {
            set_error("ktk_pool_extend: slot %d is not in use", s);
            return KTK_ERR_ARG;
        }
        if (pages_for(pool, pool->tokens[(size_t)s] + tokens_each) > pool->reserved[(size_t)s]) {
            set_error("ktk_pool_extend: slot %d would outgrow the %lld pages promised at admission", s,
                      (long long)pool->reserved[(size_t)s]);
            return KTK_ERR_TOO_LARGE;
        }
    }
    for (int32_t i = 0; i < n; ++i) {
        const size_t s = (size_t)slots[i];
        pool->tokens[s] += tokens_each;
        const int64_t need = pages_for(pool, pool->tokens[s]);
        while ((int64_t)pool->pages[s].size() < need) {      // inside the promise: the page exists
            pool->pages[s].push_back(pool->free_list.back());
            pool->free_list.pop_back();
            pool->promised -= 1;
        }
    }
    return KTK_OK;
}

extern "C" int ktk_pool_release(ktk_pool* pool, int32_t slot) {
    if (!slot_ok(pool, slot) || pool->tokens[(size_t)slot] < 0) {
        set_error("ktk_pool_release: slot %d is not in use", slot);
        return KTK_ERR_ARG;
    }
    std::vector<int32_t>& mine = pool->pages[(size_t)slot];
    pool->promised -= pool->reserved[(size_t)slot] - (int64_t)mine.size();
    for (size_t i = mine.size(); i-- > 0;) pool->free_list.push_back(mine[i]);
    mine.clear();
    pool->tokens[(size_t)slot] = -1;
    pool->reserved[(size_t)slot] = 0;
    return KTK_OK;
}

extern "C" int64_t ktk_pool_export(const ktk_pool* pool, const int32_t* slots, int32_t n, int32_t* kv_indices,
                                   int64_t indices_capacity, int32_t* kv_indptr, int32_t* kv_last_page_len) {
    if (pool == nullptr || n < 0 || (n > 0 && slots == nullptr) || kv_indptr == nullptr ||
        (n > 0 && kv_last_page_len == nullptr)) {
        set_error("ktk_pool_export: bad arguments");
        return KTK_ERR_ARG;
    }
    int64_t total = 0;
    kv_indptr[0] = 0;
    for (int32_t i = 0; i < n; ++i) {
        const int32_t s = slots[i];
        if (!slot_ok(pool, s) || pool->tokens[(size_t)s] < 0) {
            set_error("ktk_pool_export: slot %d is not in use", s);
            return KTK_ERR_ARG;
        }
        const std::vector<int32_t>& mine = pool->pages[(size_t)s];
        if (total + (int64_t)mine.size() > indices_capacity || total + (int64_t)mine.size() > 2147483647LL) {
            set_error("ktk_pool_export: kv_indices holds %lld entries, more are needed", (long long)indices_capacity);
            return KTK_ERR_TOO_LARGE;
        }
        if (!mine.empty()) std::memcpy(kv_indices + total, mine.data(), mine.size() * sizeof(int32_t));
        total += (int64_t)mine.size();
        kv_indptr[i + 1] = (int32_t)total;
        const int64_t t = pool->tokens[(size_t)s];
        kv_last_page_len[i] = (t == 0) ? 0 : (int32_t)((t - 1) % pool->page_size + 1);
    }
    return total;
}
