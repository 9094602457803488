// Shared declarations of the paged flash-decode kernels.
#pragma once

#include "ktk_common.cuh"

namespace ktk {

// What one decode launch needs.  `entries` is either the selected-page table
// [B, Hkv, topk+1] (sparse, topk >= 1) or the CSR page list kv_indices (dense,
// topk < 0): both are lists of physical page ids whose last element is the page
// being filled.
struct DecodeParams {
    const void* q;
    const void* cache;
    void* o;
    const int32_t* entries;
    const int32_t* kv_indptr;
    const int32_t* kv_last_page_len;
    int topk;
    int entry_stride;     // sparse: ints per (b, h) row of `entries`
    int batch;
    int Hkv;
    int64_t num_pages;
    float scale_log2;     // sm_scale * log2(e): softmax runs in base 2
    int num_splits;
    float* ws_ml;         // [B*Hq, S, 2]   running max (log2 domain), normaliser
    float* ws_o;          // [B*Hq, S, D]   un-normalised partial outputs
    int32_t* status;
    // view of the page table (see ktk_view in ktk.h); defaults: 0, 1, null
    int sink_tokens;             // > 0: logical page 0 holds only this many tokens and is always attended
    int local_tokens;            // the newest tokens that are always attended
    const int32_t* page_count;   // non-null: pages of sequence b (kv_indptr[b] is then only the start)
};

constexpr float kLog2e = 1.4426950408889634f;

// How the pages of one sequence split into always-attended and scored ones.
//   front : 1 if logical page 0 is a short "sink" page (sink_tokens > 0), else 0
//   n_dyn : scored pages, logical [front, front + n_dyn) -- every full page whose tokens all lie
//           more than `local_tokens` behind the end of the sequence
//   back  : pages after them, always attended (the page being filled is among them)
struct PageSplit {
    int n_pages, front, n_dyn, back, last;
    bool bad;
};

__device__ __forceinline__ PageSplit page_split(const int32_t* kv_indptr, const int32_t* page_count,
                                                const int32_t* kv_last_page_len, int b, int sink_tokens,
                                                int local_tokens) {
    PageSplit ps;
    ps.n_pages = page_count ? page_count[b] : kv_indptr[b + 1] - kv_indptr[b];
    ps.last = (ps.n_pages > 0) ? kv_last_page_len[b] : kPageSize;
    ps.bad = ps.n_pages > 0 && (ps.last < 1 || ps.last > kPageSize);
    ps.front = (sink_tokens > 0 && ps.n_pages > 0) ? 1 : 0;
    const int n_after = ps.n_pages - ps.front;
    const int len_after = (n_after > 0) ? (n_after - 1) * kPageSize + ps.last : 0;
    const int dyn_tokens = len_after - local_tokens;
    ps.n_dyn = (dyn_tokens > 0) ? dyn_tokens / kPageSize : 0;
    ps.back = n_after - ps.n_dyn;
    return ps;
}

// Page list of (b, h): pointer, number of entries, tokens in the first and last entry.
struct EntryList {
    const int32_t* ptr;
    int cnt;
    int first;   // tokens in entry 0 (a sink page is short)
    int last;    // tokens in entry cnt-1
};

__device__ __forceinline__ EntryList entry_list(const DecodeParams& p, int b, int h, bool& bad) {
    EntryList e;
    const PageSplit ps = page_split(p.kv_indptr, p.page_count, p.kv_last_page_len, b, p.sink_tokens,
                                    p.local_tokens);
    bad = ps.bad;
    e.last = ps.last;
    e.first = ps.front ? p.sink_tokens : kPageSize;
    if (ps.n_pages <= 0 || bad) {
        e.ptr = nullptr;
        e.cnt = 0;
        return e;
    }
    if (p.topk >= 0) {
        e.cnt = ps.front + (ps.n_dyn < p.topk ? ps.n_dyn : p.topk) + ps.back;
        e.ptr = p.entries + ((int64_t)b * p.Hkv + h) * p.entry_stride;
    } else {
        e.cnt = ps.n_pages;
        e.ptr = p.entries + p.kv_indptr[b];
    }
    return e;
}

// tokens held by entry e of a list
__device__ __forceinline__ int entry_tokens(const EntryList& el, int e) {
    if (e == el.cnt - 1) return el.last;
    if (e == 0) return el.first;
    return kPageSize;
}

// What the page table says about sequence b: its page list, and how many tokens it holds in all.
struct SeqPages {
    int start, n_pages, last_fill, first_fill, total;
    bool bad;
};
__device__ __forceinline__ SeqPages seq_pages(const int32_t* kv_indptr, const int32_t* page_count,
                                              const int32_t* kv_last_page_len, int sink, int b) {
    SeqPages s;
    s.start = kv_indptr[b];
    s.n_pages = page_count ? page_count[b] : kv_indptr[b + 1] - kv_indptr[b];
    s.last_fill = s.n_pages > 0 ? kv_last_page_len[b] : 0;
    s.first_fill = sink > 0 ? sink : kPageSize;
    s.bad = s.n_pages < 0 || (s.n_pages > 0 && (s.last_fill < 1 || s.last_fill > kPageSize)) ||
            (sink > 0 && s.n_pages == 1 && s.last_fill > sink);
    if (s.n_pages <= 0) s.total = 0;
    else if (s.n_pages == 1) s.total = s.last_fill;
    else s.total = s.first_fill + (s.n_pages - 2) * kPageSize + s.last_fill;
    return s;
}
// position of the first token of logical page e
__device__ __forceinline__ int page_first_pos(int e, int first_fill) {
    return e == 0 ? 0 : first_fill + (e - 1) * kPageSize;
}
// pages that hold the first `visible` tokens (visible >= 1), and the tokens of the last of them
__device__ __forceinline__ void pages_for(int visible, int first_fill, int& count, int& last) {
    if (visible <= first_fill) { count = 1; last = visible; return; }
    const int behind = visible - first_fill;
    count = 1 + (behind + kPageSize - 1) / kPageSize;
    last = behind - (count - 2) * kPageSize;
}

// logical page and slot of token position `pos`
__device__ __forceinline__ void page_of_pos(int pos, int first_fill, int& e, int& slot) {
    if (pos < first_fill) { e = 0; slot = pos; return; }
    e = 1 + (pos - first_fill) / kPageSize;
    slot = (pos - first_fill) % kPageSize;
}

int launch_decode_simt(const DecodeParams& p, int dtype, int G, cudaStream_t st);
int launch_decode_mma(const DecodeParams& p, int G, cudaStream_t st);
int launch_combine(const DecodeParams& p, int dtype, int G, cudaStream_t st);
int32_t legacy_num_splits(const ktk_shape* shape, int32_t max_entries);          // per-list split count
int32_t policy_num_splits(const ktk_shape* shape, int variant, int32_t max_entries);   // what num_splits = 0 means

}  // namespace ktk
