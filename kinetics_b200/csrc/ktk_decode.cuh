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
    int batch;
    int Hkv;
    int64_t num_pages;
    float scale_log2;     // sm_scale * log2(e): softmax runs in base 2
    int num_splits;
    float* ws_ml;         // [B*Hq, S, 2]   running max (log2 domain), normaliser
    float* ws_o;          // [B*Hq, S, D]   un-normalised partial outputs
    int32_t* status;
};

constexpr float kLog2e = 1.4426950408889634f;

// Page list of (b, h): pointer, number of entries, tokens in the last entry.
struct EntryList {
    const int32_t* ptr;
    int cnt;
    int last;
};

__device__ __forceinline__ EntryList entry_list(const DecodeParams& p, int b, int h, bool& bad) {
    EntryList e;
    const int beg = p.kv_indptr[b], end = p.kv_indptr[b + 1];
    const int n_pages = end - beg;
    e.last = (n_pages > 0) ? p.kv_last_page_len[b] : kPageSize;
    bad = n_pages > 0 && (e.last < 1 || e.last > kPageSize);
    if (n_pages <= 0 || bad) {
        e.ptr = nullptr;
        e.cnt = 0;
        return e;
    }
    if (p.topk >= 0) {
        const int scored = n_pages - 1;
        e.cnt = (scored < p.topk ? scored : p.topk) + 1;
        e.ptr = p.entries + ((int64_t)b * p.Hkv + h) * (p.topk + 1);
    } else {
        e.cnt = n_pages;
        e.ptr = p.entries + beg;
    }
    return e;
}

int launch_decode_simt(const DecodeParams& p, int dtype, int G, cudaStream_t st);
int launch_decode_mma(const DecodeParams& p, int G, cudaStream_t st);
int launch_combine(const DecodeParams& p, int dtype, int G, cudaStream_t st);

}  // namespace ktk
