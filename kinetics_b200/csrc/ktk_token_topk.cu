// Token-level top-k sparsity (LiteSys/litesys/attention/sparsity_utils.py:6-21, `topk_sparsity`) and the
// paged forms of the logits and probability x value steps it sits between.
//
// The mask needs the true logit of EVERY token of the dynamic region [sink, len - local), so unlike the
// block top-k path nothing can be skipped while scoring: all keys are read.  What the selection saves is
// the value half -- only the kept tokens' value rows are read.  The chain is the reference's own
// (batch_cache.py:154-168): logits -> mask -> softmax -> probabilities x values, with the dense fp32
// logits buffer [rows, Hq, max_len] the reference also keeps.
//   token_topk_mask_kernel   per (row, kv head): mean logit over the query group, the topk largest tokens of
//                            the dynamic region stay (radix select over order-preserving keys in shared
//                            memory, ties to the lower position), the rest becomes -inf for every head of the group
//   paged_qk_kernel          logits of one query row against the keys of its pages, read through the page table
//   paged_sv_kernel          sum of p * V over the positions whose probability is not zero
#include "ktk_decode.cuh"

namespace ktk {

constexpr int kTokThreads = 256;
constexpr int kTokMaxDynamic = 49152;        // keys of the dynamic region live in shared memory (4 B each)

__global__ void __launch_bounds__(kTokThreads)
token_topk_mask_kernel(float* __restrict__ logits, const int32_t* __restrict__ offset, int Hq, int Hkv,
                       int64_t max_len, int topk, int local, int sink, int32_t* status) {
    extern __shared__ uint32_t keys[];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_want;
    __shared__ uint32_t tie_count[kTokThreads];
    const int b = blockIdx.x, h = blockIdx.y;
    const int G = Hq / Hkv;
    int64_t len = offset[b];
    if (len > max_len) len = max_len;
    if (len <= (int64_t)sink + topk + local) return;            // sparsity_utils.py:9,12: short rows stay dense
    const int n_dyn = (int)(len - local - sink);
    if (n_dyn > kTokMaxDynamic) {
        if (threadIdx.x == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    float* base = logits + ((int64_t)b * Hq + (int64_t)h * G) * max_len + sink;
    for (int s = threadIdx.x; s < n_dyn; s += kTokThreads) {
        float m = 0.0f;
        for (int g = 0; g < G; ++g) m += base[(int64_t)g * max_len + s];
        keys[s] = score_to_key(m / (float)G);
    }
    if (threadIdx.x == 0) { s_prefix = 0; s_want = (uint32_t)topk; }
    __syncthreads();
    // the topk-th largest key, one byte at a time from the top
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[threadIdx.x] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (int s = threadIdx.x; s < n_dyn; s += kTokThreads) {
            const uint32_t k = keys[s];
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t want = s_want, above = 0;
            int bin = 255;
            for (; bin > 0; --bin) {
                if (above + hist[bin] >= want) break;
                above += hist[bin];
            }
            s_want = want - above;                  // how many of this bin are still to be taken
            s_prefix = prefix | ((uint32_t)bin << shift);
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t kth = s_prefix;                  // keys above it are kept; of the keys equal to it, the first s_want
    const uint32_t want_ties = s_want;
    // ties in position order: every thread owns a contiguous range
    const int chunk = (n_dyn + kTokThreads - 1) / kTokThreads;
    const int lo = threadIdx.x * chunk;
    const int hi = lo + chunk < n_dyn ? lo + chunk : n_dyn;
    uint32_t mine = 0;
    for (int s = lo; s < hi; ++s) mine += keys[s] == kth ? 1u : 0u;
    tie_count[threadIdx.x] = mine;
    __syncthreads();
    uint32_t before = 0;
    for (int t = 0; t < (int)threadIdx.x; ++t) before += tie_count[t];
    for (int s = lo; s < hi; ++s) {
        const uint32_t k = keys[s];
        bool keep = k > kth;
        if (k == kth) { keep = before < want_ties; ++before; }
        if (!keep)
            for (int g = 0; g < G; ++g) base[(int64_t)g * max_len + s] = -INFINITY;
    }
}

struct PagedChainParams {
    const void* cache;
    const int32_t* kv_indices;
    const int32_t* kv_indptr;
    const int32_t* kv_last_page_len;
    const int32_t* page_count;
    int sink_tokens;
    int Hkv, G;
    int64_t num_pages, max_len;
    int32_t* status;
};

// address of the K (which = 0) or V (which = 1) row of token `pos` of a sequence; null if the page id is bad
template <typename T>
__device__ __forceinline__ const T* paged_row(const PagedChainParams& p, const SeqPages& sp, int pos, int h, int which) {
    int e, slot;
    page_of_pos(pos, sp.first_fill, e, slot);
    const int64_t page = p.kv_indices[sp.start + e];
    if (page < 0 || page >= p.num_pages) { report(p.status, KTK_STATUS_BAD_PAGE); return nullptr; }
    return (const T*)p.cache + (((page * 2 + which) * kPageSize + slot) * p.Hkv + h) * (int64_t)kHeadDim;
}

// logits[row, h*G+g, s] = scale * q[row, h*G+g, :] . K[s, :] for s < tokens(row).  One CTA per (row, kv head,
// 256 positions); a half-warp per position, lane j of it owns elements 8j..8j+7.
template <typename T>
__global__ void __launch_bounds__(kTokThreads)
paged_qk_kernel(const T* __restrict__ q, const PagedChainParams p, float* __restrict__ logits, float scale) {
    const int b = blockIdx.x, h = blockIdx.y;
    const SeqPages sp = seq_pages(p.kv_indptr, p.page_count, p.kv_last_page_len, p.sink_tokens, b);
    if (sp.bad) { if (threadIdx.x == 0 && blockIdx.z == 0) report(p.status, KTK_STATUS_BAD_TABLE); return; }
    const int len = sp.total < p.max_len ? sp.total : (int)p.max_len;
    const int half = threadIdx.x >> 4, j = threadIdx.x & 15;
    const int G = p.G, Hq = p.Hkv * G;
    float qv[8][8];
#pragma unroll
    for (int g = 0; g < 8; ++g)
        if (g < G) load8(q + ((int64_t)b * Hq + (int64_t)h * G + g) * kHeadDim + 8 * j, qv[g]);
    float* out = logits + ((int64_t)b * Hq + (int64_t)h * G) * p.max_len;
    const int s0 = blockIdx.z * kTokThreads;
    for (int i = 0; i < 16; ++i) {                 // the same trip count for every lane: the shuffles below need all 32
        const int s = s0 + half + i * (kTokThreads / 16);
        const bool valid = s < len;
        const T* krow = valid ? paged_row<T>(p, sp, s, h, 0) : nullptr;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (krow != nullptr) load8(krow + 8 * j, x);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            if (g < G) {
                float d = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) d = fmaf(qv[g][e], x[e], d);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o, 16);
                if (valid && j == 0) out[(int64_t)g * p.max_len + s] = d * scale;
            }
        }
    }
}

// out[row, h*G+g, :] = sum over s < tokens(row) of p[row, h*G+g, s] * V[s, :]; positions whose probability is
// zero for every head of the group (the masked ones) are not read.  One CTA per (row, kv head).
template <typename T>
__global__ void __launch_bounds__(kTokThreads)
paged_sv_kernel(const PagedChainParams p, const float* __restrict__ probs, T* __restrict__ out) {
    constexpr int kHalves = kTokThreads / 16;
    __shared__ float red[kHalves][kHeadDim];
    const int b = blockIdx.x, h = blockIdx.y;
    const SeqPages sp = seq_pages(p.kv_indptr, p.page_count, p.kv_last_page_len, p.sink_tokens, b);
    if (sp.bad) { if (threadIdx.x == 0) report(p.status, KTK_STATUS_BAD_TABLE); return; }
    const int len = sp.total < p.max_len ? sp.total : (int)p.max_len;
    const int half = threadIdx.x >> 4, j = threadIdx.x & 15;
    const int G = p.G, Hq = p.Hkv * G;
    const float* pbase = probs + ((int64_t)b * Hq + (int64_t)h * G) * p.max_len;
    float acc[8][8];
#pragma unroll
    for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
    for (int s = half; s < len; s += kHalves) {
        float pg[8];
        bool any = false;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            pg[g] = g < G ? pbase[(int64_t)g * p.max_len + s] : 0.0f;
            any = any || pg[g] != 0.0f;
        }
        if (!any) continue;                         // uniform over the half-warp
        const T* vrow = paged_row<T>(p, sp, s, h, 1);
        if (vrow == nullptr) continue;
        float x[8];
        load8(vrow + 8 * j, x);
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pg[g], x[e], acc[g][e]);
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if (g >= G) break;
        __syncthreads();                            // `red` of the previous head has been read
#pragma unroll
        for (int e = 0; e < 8; ++e) red[half][8 * j + e] = acc[g][e];
        __syncthreads();
        if (threadIdx.x < kHeadDim) {
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < kHalves; ++w) tot += red[w][threadIdx.x];
            out[((int64_t)b * Hq + (int64_t)h * G + g) * kHeadDim + threadIdx.x] = from_f32<T>(tot);
        }
    }
}

}  // namespace ktk

using namespace ktk;

extern "C" int ktk_token_topk_mask(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                                   int32_t num_kv_heads, int64_t max_len, int32_t topk, int32_t local, int32_t sink,
                                   int32_t* status, void* stream) {
    if (rows < 0 || num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads != 0 || max_len <= 0 ||
        topk < 1 || local < 0 || sink < 0) {
        set_error("ktk_token_topk_mask: bad sizes rows=%d heads=%d/%d max_len=%lld topk=%d local=%d sink=%d", rows,
                  num_q_heads, num_kv_heads, (long long)max_len, topk, local, sink);
        return KTK_ERR_ARG;
    }
    if (rows == 0) return KTK_OK;
    if (!logits || !offset) { set_error("ktk_token_topk_mask: null pointer argument"); return KTK_ERR_ARG; }
    if (num_kv_heads > 65535 || num_q_heads / num_kv_heads > 8) {
        set_error("ktk_token_topk_mask: group size <= 8 and <= 65535 kv heads are built");
        return KTK_ERR_UNSUPPORTED;
    }
    int64_t dyn = max_len - sink - local;
    if (dyn < 1) return KTK_OK;                     // no row can be longer than sink + topk + local
    if (dyn > kTokMaxDynamic) {
        set_error("ktk_token_topk_mask: a dynamic region of up to %lld tokens exceeds the %d that fit shared memory",
                  (long long)dyn, kTokMaxDynamic);
        return KTK_ERR_TOO_LARGE;
    }
    const int smem = (int)dyn * (int)sizeof(uint32_t);
    KTK_CUDA_TRY(cudaFuncSetAttribute(token_topk_mask_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "ktk_token_topk_mask");
    token_topk_mask_kernel<<<dim3((unsigned)rows, (unsigned)num_kv_heads), kTokThreads, smem, (cudaStream_t)stream>>>(
        logits, offset, num_q_heads, num_kv_heads, max_len, topk, local, sink, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_token_topk_mask");
    return KTK_OK;
}

namespace {
int paged_chain_params(const char* who, PagedChainParams& p, const void* kv_cache, const int32_t* kv_indices,
                       const int32_t* kv_indptr, const int32_t* kv_last_page_len, const ktk_view* view_in,
                       int64_t max_len, const ktk_shape* s, int32_t* status) {
    int rc = check_shape(s, who);
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, who);
    if (rc != KTK_OK) return rc;
    if (!kv_cache || !kv_indices || !kv_indptr || !kv_last_page_len || max_len <= 0) {
        set_error("%s: null pointer argument or max_len <= 0", who);
        return KTK_ERR_ARG;
    }
    if (s->group_size > 8 || s->num_kv_heads > 65535) {
        set_error("%s: group size <= 8 and <= 65535 kv heads are built", who);
        return KTK_ERR_UNSUPPORTED;
    }
    const View view = make_view(view_in);
    p.cache = kv_cache; p.kv_indices = kv_indices; p.kv_indptr = kv_indptr; p.kv_last_page_len = kv_last_page_len;
    p.page_count = view.page_count; p.sink_tokens = view.sink_tokens; p.Hkv = s->num_kv_heads; p.G = s->group_size;
    p.num_pages = s->num_pages; p.max_len = max_len; p.status = status;
    return KTK_OK;
}
}  // namespace

extern "C" int ktk_paged_qk(const void* q, const void* kv_cache, const int32_t* kv_indices, const int32_t* kv_indptr,
                            const int32_t* kv_last_page_len, const ktk_view* view, float sm_scale, float* logits,
                            int64_t max_len, const ktk_shape* s, int32_t* status, void* stream) {
    PagedChainParams p;
    int rc = paged_chain_params("ktk_paged_qk", p, kv_cache, kv_indices, kv_indptr, kv_last_page_len, view, max_len, s,
                                status);
    if (rc != KTK_OK) return rc;
    if (s->batch == 0) return KTK_OK;
    if (!q || !logits) { set_error("ktk_paged_qk: null pointer argument"); return KTK_ERR_ARG; }
    const int64_t chunks = (max_len + kTokThreads - 1) / kTokThreads;
    if (chunks > 65535) { set_error("ktk_paged_qk: max_len %lld too long", (long long)max_len); return KTK_ERR_TOO_LARGE; }
    const dim3 grid((unsigned)s->batch, (unsigned)s->num_kv_heads, (unsigned)chunks);
    cudaStream_t st = (cudaStream_t)stream;
    if (s->dtype == KTK_F32)
        paged_qk_kernel<float><<<grid, kTokThreads, 0, st>>>((const float*)q, p, logits, sm_scale);
    else
        paged_qk_kernel<__nv_bfloat16><<<grid, kTokThreads, 0, st>>>((const __nv_bfloat16*)q, p, logits, sm_scale);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_paged_qk");
    return KTK_OK;
}

extern "C" int ktk_paged_sv(const void* kv_cache, const int32_t* kv_indices, const int32_t* kv_indptr,
                            const int32_t* kv_last_page_len, const ktk_view* view, const float* probs, int64_t max_len,
                            void* out, const ktk_shape* s, int32_t* status, void* stream) {
    PagedChainParams p;
    int rc = paged_chain_params("ktk_paged_sv", p, kv_cache, kv_indices, kv_indptr, kv_last_page_len, view, max_len, s,
                                status);
    if (rc != KTK_OK) return rc;
    if (s->batch == 0) return KTK_OK;
    if (!probs || !out) { set_error("ktk_paged_sv: null pointer argument"); return KTK_ERR_ARG; }
    const dim3 grid((unsigned)s->batch, (unsigned)s->num_kv_heads);
    cudaStream_t st = (cudaStream_t)stream;
    if (s->dtype == KTK_F32)
        paged_sv_kernel<float><<<grid, kTokThreads, 0, st>>>(p, probs, (float*)out);
    else
        paged_sv_kernel<__nv_bfloat16><<<grid, kTokThreads, 0, st>>>(p, probs, (__nv_bfloat16*)out);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_paged_sv");
    return KTK_OK;
}
