// Interface between the prefill dispatcher (ktk_prefill.cu) and the tcgen05 prefill kernel (ktk_prefill_umma.cu).
#pragma once

#include "ktk_common.cuh"

namespace ktk {

struct PrefillUmmaParams {
    const void* q;
    void* o;
    const void* cache;
    const int32_t* q_indptr;
    const int32_t* kv_indices;
    const int32_t* kv_indptr;
    const int32_t* kv_last_page_len;
    const int32_t* page_count;
    int sink_tokens;
    int batch, Hkv, G;
    int64_t num_pages;
    float scale_log2;
    int32_t* status;
};

// Descriptor of the V operand (MN-major: 64 keys x 128 B rows per 64-dim tile, 128-byte swizzle): byte distance
// between the two 64-dim tiles, and between groups of eight keys.
constexpr uint32_t kUmVLbo = 64 * 128;
constexpr uint32_t kUmVSbo = 1024;

int launch_prefill_umma(const PrefillUmmaParams& p, int max_new_tokens, cudaStream_t st);

}  // namespace ktk
