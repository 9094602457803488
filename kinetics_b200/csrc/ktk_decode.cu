// Paged flash-decode attention, fp32-FMA variant, plus the split combine and
// the C entry points of the sparse (selected pages) and dense (all pages) decode.
//
// Work decomposition: one CTA of four warps per (sequence, kv head, split).
// Each warp walks its own pages (warp w takes entries w, w+4, ...) with an
// online softmax; a lane owns four consecutive head-dim elements, so a K or V
// row is one coalesced 256-byte (bf16) warp load straight from HBM, and the
// next page of the warp is already in flight in registers while the current
// one is being reduced.  The four warps merge through shared memory.
#include "ktk_decode_mma.cuh"

namespace ktk {

template <typename T> struct Raw4;
template <> struct Raw4<float> { using type = float4; };
template <> struct Raw4<__nv_bfloat16> { using type = uint2; };

__device__ __forceinline__ void cvt4(const float4& r, float (&f)[4]) {
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
}
__device__ __forceinline__ void cvt4(const uint2& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
}

constexpr int kSimtWarps = 4;

// One halving step of the warp reduce-scatter: 2W live values become W, the
// partner lane (xor 2W) receives the other half.
template <int W>
__device__ __forceinline__ void halve(float (&part)[kPageSize], int lane) {
    constexpr int off = 2 * W;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < W; ++i) {
        const float lo = part[i], hi = part[i + W];
        const float send = upper ? lo : hi;
        const float keep = upper ? hi : lo;
        part[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
}

template <typename T, int G>
__global__ void __launch_bounds__(kSimtWarps * 32)
decode_simt_kernel(const DecodeParams p) {
    using R = typename Raw4<T>::type;
    constexpr bool kPrefetch = sizeof(T) == 2;   // a page is 64 registers in bf16, 128 in fp32
    __shared__ __align__(16) float p_sm[kSimtWarps][kPageSize * G];   // probabilities [t][g]
    __shared__ __align__(16) float red_o[kSimtWarps][G][kHeadDim];
    __shared__ float red_m[kSimtWarps][G], red_l[kSimtWarps][G];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = p.num_splits;
    const int64_t bh = blockIdx.x / S;
    const int split = blockIdx.x % S;
    const int b = (int)(bh / p.Hkv), h = (int)(bh % p.Hkv);
    const int Hq = p.Hkv * G;

    bool bad;
    const EntryList el = entry_list(p, b, h, bad);
    if (bad && tid == 0 && split == 0) report(p.status, KTK_STATUS_BAD_TABLE);
    const int per = (el.cnt + S - 1) / S;
    const int e0 = split * per;
    const int e1 = (e0 + per < el.cnt) ? e0 + per : el.cnt;

    float qr[G][4];
    {
        const T* qp = (const T*)p.q + ((int64_t)b * Hq + (int64_t)h * G) * kHeadDim + lane * 4;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            load4(qp + g * kHeadDim, qr[g]);
#pragma unroll
            for (int i = 0; i < 4; ++i) qr[g][i] *= p.scale_log2;
        }
    }
    float m[G], l[G], o[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) o[g][i] = 0.0f;
    }

    const int64_t row = (int64_t)p.Hkv * kHeadDim;   // elements between consecutive tokens
    const T* cache = (const T*)p.cache;

    auto fetch = [&](int e, R (&kr)[kPageSize], R (&vr)[kPageSize]) -> bool {
        const int64_t page = el.ptr[e];
        if (page < 0 || page >= p.num_pages) {
            if (lane == 0) report(p.status, KTK_STATUS_BAD_PAGE);
            return false;
        }
        const T* kp = cache + (page * 2) * kPageSize * row + (int64_t)h * kHeadDim + lane * 4;
        const T* vp = kp + kPageSize * row;
#pragma unroll
        for (int t = 0; t < kPageSize; ++t) kr[t] = __ldg(reinterpret_cast<const R*>(kp + t * row));
#pragma unroll
        for (int t = 0; t < kPageSize; ++t) vr[t] = __ldg(reinterpret_cast<const R*>(vp + t * row));
        return true;
    };

    // one page of the warp: scores, online softmax, weighted values
    auto consume = [&](int e, const R (&kr)[kPageSize], const R (&vr)[kPageSize]) {
        const int ntok = entry_tokens(el, e);
        const int tok = lane >> 1;               // the token this lane ends up holding
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float part[kPageSize];
#pragma unroll
            for (int t = 0; t < kPageSize; ++t) {
                float kf[4];
                cvt4(kr[t], kf);
                part[t] = qr[g][0] * kf[0] + qr[g][1] * kf[1] + qr[g][2] * kf[2] + qr[g][3] * kf[3];
            }
            // reduce over the 32 lanes while scattering tokens: after the four
            // halving steps lane L holds token L>>1, the last step joins the pair
            halve<8>(part, lane);
            halve<4>(part, lane);
            halve<2>(part, lane);
            halve<1>(part, lane);
            part[0] += __shfl_xor_sync(0xffffffffu, part[0], 1);
            s[g] = (tok < ntok) ? part[0] : -INFINITY;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mx = s[g];
#pragma unroll
            for (int off = 16; off >= 2; off >>= 1)
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[g], mx);      // finite: token 0 is always valid
            const float alpha = exp2f(m[g] - m_new);
            const float pr = exp2f(s[g] - m_new);
            float sum = pr;
#pragma unroll
            for (int off = 16; off >= 2; off >>= 1)
                sum += __shfl_xor_sync(0xffffffffu, sum, off);
            m[g] = m_new;
            l[g] = l[g] * alpha + sum;
#pragma unroll
            for (int i = 0; i < 4; ++i) o[g][i] *= alpha;
            if ((lane & 1) == 0) p_sm[warp][tok * G + g] = pr;
        }
        __syncwarp();
#pragma unroll
        for (int t = 0; t < kPageSize; ++t) {
            if (t < ntok) {       // rows past the fill level may hold anything
                float vf[4];
                cvt4(vr[t], vf);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pg = p_sm[warp][t * G + g];
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[g][i] = fmaf(pg, vf[i], o[g][i]);
                }
            }
        }
        __syncwarp();
    };

    if constexpr (kPrefetch) {
        // two register buffers, alternated: the warp's next page is in flight
        // while the current one is reduced
        R ka[kPageSize], va[kPageSize], kb[kPageSize], vb[kPageSize];
        int e = e0 + warp;
        bool have_a = (e < e1) ? fetch(e, ka, va) : false;
        while (e < e1) {
            const int en = e + kSimtWarps;
            const bool have_b = (en < e1) ? fetch(en, kb, vb) : false;
            if (have_a) consume(e, ka, va);
            if (en >= e1) break;
            const int enn = en + kSimtWarps;
            have_a = (enn < e1) ? fetch(enn, ka, va) : false;
            if (have_b) consume(en, kb, vb);
            e = enn;
        }
    } else {
        R ka[kPageSize], va[kPageSize];
        for (int e = e0 + warp; e < e1; e += kSimtWarps)
            if (fetch(e, ka, va)) consume(e, ka, va);
    }

    // ---- merge the four warps ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
        *reinterpret_cast<float4*>(&red_o[warp][g][lane * 4]) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
    }
    __syncthreads();
    const int d = tid;   // 128 threads, one per head-dim element
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float M = red_m[0][g];
#pragma unroll
        for (int w = 1; w < kSimtWarps; ++w) M = fmaxf(M, red_m[w][g]);
        float L = 0.0f, O = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kSimtWarps; ++w) {
                const float wt = exp2f(red_m[w][g] - M);
                L += wt * red_l[w][g];
                O += wt * red_o[w][g][d];
            }
        }
        const int64_t qh = (int64_t)b * Hq + (int64_t)h * G + g;
        if (S == 1) {
            ((T*)p.o)[qh * kHeadDim + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
        } else {
            p.ws_o[(qh * S + split) * kHeadDim + d] = O;
            if (d == 0) {
                p.ws_ml[(qh * S + split) * 2 + 0] = M;
                p.ws_ml[(qh * S + split) * 2 + 1] = L;
            }
        }
    }
}

// One CTA per (sequence, query head): merges the S partials of a split decode.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
combine_kernel(const float* __restrict__ ws_ml, const float* __restrict__ ws_o, T* __restrict__ o,
               int S) {
    const int64_t qh = blockIdx.x;
    const int d = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, ws_ml[(qh * S + s) * 2]);
    float L = 0.0f, O = 0.0f;
    if (M != -INFINITY) {
        for (int s = 0; s < S; ++s) {
            const float ms = ws_ml[(qh * S + s) * 2];
            if (ms == -INFINITY) continue;         // empty split: its partial row is unspecified
            const float wt = exp2f(ms - M);
            L += wt * ws_ml[(qh * S + s) * 2 + 1];
            O += wt * ws_o[(qh * S + s) * kHeadDim + d];
        }
    }
    o[qh * kHeadDim + d] = from_f32<T>(L > 0.0f ? O / L : 0.0f);
}

template <typename T, int G>
static int simt_launch(const DecodeParams& p, cudaStream_t st) {
    const int64_t ctas = (int64_t)p.batch * p.Hkv * p.num_splits;
    decode_simt_kernel<T, G><<<(unsigned)ctas, kSimtWarps * 32, 0, st>>>(p);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk decode (simt)");
    return KTK_OK;
}

template <typename T>
static int simt_group(const DecodeParams& p, int G, cudaStream_t st) {
    switch (G) {
        case 1: return simt_launch<T, 1>(p, st);
        case 2: return simt_launch<T, 2>(p, st);
        case 4: return simt_launch<T, 4>(p, st);
        default: return simt_launch<T, 8>(p, st);
    }
}

int launch_decode_simt(const DecodeParams& p, int dtype, int G, cudaStream_t st) {
    return dtype == KTK_F32 ? simt_group<float>(p, G, st) : simt_group<__nv_bfloat16>(p, G, st);
}

int launch_combine(const DecodeParams& p, int dtype, int G, cudaStream_t st) {
    const int64_t rows = (int64_t)p.batch * p.Hkv * G;
    if (dtype == KTK_F32)
        combine_kernel<float><<<(unsigned)rows, kHeadDim, 0, st>>>(p.ws_ml, p.ws_o, (float*)p.o, p.num_splits);
    else
        combine_kernel<__nv_bfloat16><<<(unsigned)rows, kHeadDim, 0, st>>>(p.ws_ml, p.ws_o, (__nv_bfloat16*)p.o, p.num_splits);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk decode (combine)");
    return KTK_OK;
}

static int decode_common(const char* who, const void* q, const void* cache, const int32_t* entries,
                         int topk, int max_entries, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, float sm_scale, void* o, void* workspace,
                         size_t workspace_bytes, int num_splits, int variant, const ktk_shape* s,
                         int32_t* status, void* stream, const ktk_view* view_in = nullptr,
                         int row_width = 0) {
    int rc = check_shape(s, who);
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, who);
    if (rc != KTK_OK) return rc;
    const View view = make_view(view_in);
    if (topk >= 0) {
        const int need_width = view_row_width(topk, view);
        if (row_width == 0) row_width = need_width;
        if (row_width < need_width) {
            set_error("%s: selected-page rows of %d entries, this view needs %d", who, row_width, need_width);
            return KTK_ERR_ARG;
        }
    }
    if (s->batch == 0) return KTK_OK;
    if (!q || !cache || !entries || !kv_indptr || !kv_last_page_len || !o) {
        set_error("%s: null pointer argument", who);
        return KTK_ERR_ARG;
    }
    if (num_splits < KTK_SPLITS_BALANCED || num_splits > 256) {
        set_error("%s: num_splits %d outside [0, 256] and not KTK_SPLITS_BALANCED", who, num_splits);
        return KTK_ERR_ARG;
    }
    if (variant != KTK_VARIANT_AUTO && variant != KTK_VARIANT_SIMT && variant != KTK_VARIANT_MMA) {
        set_error("%s: unknown variant %d", who, variant);
        return KTK_ERR_ARG;
    }
    if (variant == KTK_VARIANT_MMA && s->dtype != KTK_BF16) {
        set_error("%s: the tensor-core variant is bf16 only", who);
        return KTK_ERR_UNSUPPORTED;
    }
    const bool tensor_cores = s->dtype == KTK_BF16 && variant != KTK_VARIANT_SIMT;
    if (num_splits == KTK_SPLITS_BALANCED && !tensor_cores) {
        set_error("%s: the balanced partition exists for the bf16 tensor-core variant only", who);
        return KTK_ERR_UNSUPPORTED;
    }
    if (num_splits == 0) num_splits = policy_num_splits(s, variant, max_entries);
    const bool balanced = num_splits == KTK_SPLITS_BALANCED;
    const int64_t ctas = balanced ? 1 : (int64_t)s->batch * s->num_kv_heads * num_splits;
    if (ctas > 2147483647LL) {
        set_error("%s: batch * num_kv_heads * num_splits exceeds the grid limit", who);
        return KTK_ERR_TOO_LARGE;
    }
    DecodeParams p;
    p.q = q; p.cache = cache; p.o = o; p.entries = entries;
    p.kv_indptr = kv_indptr; p.kv_last_page_len = kv_last_page_len;
    p.sink_tokens = view.sink_tokens; p.local_tokens = view.local_tokens; p.page_count = view.page_count;
    p.entry_stride = row_width;
    p.topk = topk; p.batch = s->batch; p.Hkv = s->num_kv_heads; p.num_pages = s->num_pages;
    p.scale_log2 = sm_scale * kLog2e;
    p.num_splits = num_splits; p.ws_ml = nullptr; p.ws_o = nullptr; p.status = status;
    if (num_splits > 1 || balanced) {
        const size_t need = ktk_decode_workspace_bytes(s, num_splits);
        if (workspace == nullptr || workspace_bytes < need) {
            set_error("%s: workspace of %zu bytes needed for %d splits, got %zu", who, need,
                      num_splits, workspace ? workspace_bytes : (size_t)0);
            return KTK_ERR_WORKSPACE;
        }
        const int64_t rows = balanced ? (int64_t)(need / ((2 + kHeadDim) * sizeof(float)))
                                      : (int64_t)s->batch * s->num_kv_heads * s->group_size * num_splits;
        p.ws_ml = (float*)workspace;
        p.ws_o = (float*)workspace + rows * 2;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (balanced)
        return launch_decode_stream(p, s->group_size, topk >= 0 ? row_width : max_entries, st);
    if (variant == KTK_VARIANT_AUTO)
        variant = (s->dtype == KTK_BF16) ? KTK_VARIANT_MMA : KTK_VARIANT_SIMT;
    if (variant == KTK_VARIANT_MMA)
        rc = launch_decode_mma(p, s->group_size, st);
    else
        rc = launch_decode_simt(p, s->dtype, s->group_size, st);
    if (rc != KTK_OK) return rc;
    if (num_splits > 1) rc = launch_combine(p, s->dtype, s->group_size, st);
    return rc;
}

}  // namespace ktk

using namespace ktk;

extern "C" int32_t ktk_decode_num_splits(const ktk_shape* shape, int32_t max_entries) {
    if (shape != nullptr && shape->dtype == KTK_BF16) return KTK_SPLITS_BALANCED;
    return legacy_num_splits(shape, max_entries);
}

int32_t ktk::policy_num_splits(const ktk_shape* shape, int variant, int32_t max_entries) {
    const bool tensor_cores = shape != nullptr && shape->dtype == KTK_BF16 && variant != KTK_VARIANT_SIMT;
    return tensor_cores ? KTK_SPLITS_BALANCED : legacy_num_splits(shape, max_entries);
}

int32_t ktk::legacy_num_splits(const ktk_shape* shape, int32_t max_entries) {
    if (shape == nullptr || shape->batch <= 0 || shape->num_kv_heads <= 0 || max_entries <= 0) return 1;
    // enough CTAs for four per SM, but never fewer than 8 pages per split
    const int64_t items = (int64_t)shape->batch * shape->num_kv_heads;
    const int64_t target = 4LL * sm_count();
    int64_t s = (target + items - 1) / items;
    const int64_t cap = (max_entries + 7) / 8;
    if (s > cap) s = cap;
    if (s > 64) s = 64;
    if (s < 1) s = 1;
    return (int32_t)s;
}

extern "C" size_t ktk_decode_workspace_bytes(const ktk_shape* shape, int32_t num_splits) {
    if (shape != nullptr && num_splits == KTK_SPLITS_BALANCED) return stream_workspace_bytes(shape->group_size);
    if (shape == nullptr || num_splits <= 1) return 0;
    const size_t rows = (size_t)shape->batch * shape->num_kv_heads * shape->group_size * num_splits;
    return rows * (2 + kHeadDim) * sizeof(float);
}

extern "C" int ktk_sparse_decode(const void* q, const void* kv_cache, const int32_t* sel_pages,
                                 int32_t topk, const int32_t* kv_indptr,
                                 const int32_t* kv_last_page_len, float sm_scale, void* o,
                                 void* workspace, size_t workspace_bytes, int32_t num_splits,
                                 int32_t variant, const ktk_shape* shape, int32_t* status,
                                 void* stream) {
    if (topk < 1) {
        set_error("ktk_sparse_decode: topk must be >= 1 (got %d)", topk);
        return KTK_ERR_ARG;
    }
    return decode_common("ktk_sparse_decode", q, kv_cache, sel_pages, topk, topk + 1, kv_indptr,
                         kv_last_page_len, sm_scale, o, workspace, workspace_bytes, num_splits,
                         variant, shape, status, stream);
}

extern "C" int ktk_dense_decode(const void* q, const void* kv_cache, const int32_t* kv_indices,
                                const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                int32_t max_pages_per_seq, float sm_scale, void* o, void* workspace,
                                size_t workspace_bytes, int32_t num_splits, int32_t variant,
                                const ktk_shape* shape, int32_t* status, void* stream) {
    if (max_pages_per_seq < 1) max_pages_per_seq = 1;
    return decode_common("ktk_dense_decode", q, kv_cache, kv_indices, -1, max_pages_per_seq,
                         kv_indptr, kv_last_page_len, sm_scale, o, workspace, workspace_bytes,
                         num_splits, variant, shape, status, stream);
}

// ---------------------------------------------------------------------------
// Split decode without a caller-provided workspace and without any allocation.
//
// Some hosts of this library cannot hand it scratch memory and must not see it
// allocate: a serving engine that claimed all of HBM for its own KV-page pool at
// start-up (a cudaMalloc would fail or eat into that pool), or a decode loop that
// cannot afford the device-wide synchronisation an allocation implies.  For them
// the split partials live in the array below, which is part of the library image:
// every GPU that loads the library carries these 16 MiB until the process exits.
//
// g_noalloc_scratch is a device symbol.  Host code may not use its name as an
// address; ktk_noalloc_scratch() asks the runtime for the real device address, once
// per device, with that device current, and that address is what the kernels get.
// ---------------------------------------------------------------------------
#include <mutex>

namespace ktk {

constexpr size_t kNoAllocScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;

static int ktk_noalloc_scratch(void** out) {
    static std::mutex mu;
    static void* addr[kMaxDevices] = {};
    int dev = -1;
    KTK_CUDA_TRY(cudaGetDevice(&dev), "ktk_sparse_decode_noalloc");
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("ktk_sparse_decode_noalloc: device ordinal %d outside [0, %d)", dev, kMaxDevices);
        return KTK_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        KTK_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch), "ktk_sparse_decode_noalloc (scratch address)");
        addr[dev] = p;
    }
    *out = addr[dev];
    return KTK_OK;
}

}  // namespace ktk

extern "C" size_t ktk_noalloc_scratch_bytes(void) { return ktk::kNoAllocScratchBytes; }

extern "C" int ktk_sparse_decode_noalloc(const void* q, const void* kv_cache, const int32_t* sel_pages,
                                         int32_t topk, const int32_t* kv_indptr,
                                         const int32_t* kv_last_page_len, float sm_scale, void* o,
                                         int32_t num_splits, int32_t variant, const ktk_shape* shape,
                                         int32_t* status, void* stream) {
    if (topk < 1) {
        set_error("ktk_sparse_decode_noalloc: topk must be >= 1 (got %d)", topk);
        return KTK_ERR_ARG;
    }
    int rc = check_shape(shape, "ktk_sparse_decode_noalloc");
    if (rc != KTK_OK) return rc;
    if (num_splits != KTK_SPLITS_BALANCED && (num_splits < 0 || num_splits > 256)) {
        set_error("ktk_sparse_decode_noalloc: num_splits %d is neither KTK_SPLITS_BALANCED nor in [0, 256]", num_splits);
        return KTK_ERR_ARG;
    }
    if (num_splits == 0) num_splits = policy_num_splits(shape, variant, topk + 1);
    const size_t need = ktk_decode_workspace_bytes(shape, num_splits);
    if (need > kNoAllocScratchBytes) {
        set_error("ktk_sparse_decode_noalloc: %d splits of this batch need %zu bytes of scratch, the built-in "
                  "array holds %zu; use fewer splits, or ktk_sparse_decode with a workspace of your own",
                  num_splits, need, (size_t)kNoAllocScratchBytes);
        return KTK_ERR_TOO_LARGE;
    }
    void* scratch = nullptr;
    if (need > 0) {
        rc = ktk_noalloc_scratch(&scratch);
        if (rc != KTK_OK) return rc;
    }
    // Every partial slot a launch later reads is written by that same launch (an empty split
    // writes "nothing seen"), so the array needs no clearing between calls.
    return decode_common("ktk_sparse_decode_noalloc", q, kv_cache, sel_pages, topk, topk + 1, kv_indptr,
                         kv_last_page_len, sm_scale, o, scratch, need, num_splits, variant, shape, status,
                         stream);
}

extern "C" int ktk_sparse_decode_v(const void* q, const void* kv_cache, const int32_t* sel_pages,
                                   int32_t topk, const ktk_view* view, int32_t row_width,
                                   const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                   float sm_scale, void* o, void* workspace, size_t workspace_bytes,
                                   int32_t num_splits, int32_t variant, const ktk_shape* shape,
                                   int32_t* status, void* stream) {
    if (topk < 1) {
        set_error("ktk_sparse_decode_v: topk must be >= 1 (got %d)", topk);
        return KTK_ERR_ARG;
    }
    if (check_view(view, "ktk_sparse_decode_v") != KTK_OK) return KTK_ERR_ARG;
    return decode_common("ktk_sparse_decode_v", q, kv_cache, sel_pages, topk,
                         view_row_width(topk, make_view(view)), kv_indptr, kv_last_page_len, sm_scale, o,
                         workspace, workspace_bytes, num_splits, variant, shape, status, stream, view,
                         row_width);
}

extern "C" int ktk_dense_decode_v(const void* q, const void* kv_cache, const int32_t* kv_indices,
                                  const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                  const ktk_view* view, int32_t max_pages_per_seq, float sm_scale, void* o,
                                  void* workspace, size_t workspace_bytes, int32_t num_splits,
                                  int32_t variant, const ktk_shape* shape, int32_t* status, void* stream) {
    if (max_pages_per_seq < 1) max_pages_per_seq = 1;
    return decode_common("ktk_dense_decode_v", q, kv_cache, kv_indices, -1, max_pages_per_seq, kv_indptr,
                         kv_last_page_len, sm_scale, o, workspace, workspace_bytes, num_splits, variant,
                         shape, status, stream, view, 0);
}
