// GQA query x page-summary scoring fused with per-(sequence, kv head) top-k
// page selection.  HBM-bound: one streaming pass over the sequence's summaries
// (n_scored * D elements), everything else stays in shared memory.
//
// The arithmetic order of a score is part of the contract (selection must be
// bit-exact against the CPU oracle):
//   qbar[d]  = (q[g=0][d] + q[1][d] + ... + q[G-1][d]) * (1/G)      fp32, in g order
//   lane j of a 16-lane group owns elements 8j..8j+7 of the summary row:
//   part_j   = fma(qbar[8j+7], s[8j+7], ... fma(qbar[8j], s[8j], 0))   in element order
//   then four butterfly steps part_j += part_(j xor off), off = 8, 4, 2, 1
//   score    = part_0 + 0.0f
// Selection orders pages by the 48-bit composite (key(score) << 16) | (0xFFFF - page),
// which is unique per page: the k largest composites are "largest score first, ties
// to the lowest page number".
#include "ktk_common.cuh"

namespace ktk {

constexpr int kSelThreads = 256;
constexpr int kSelUnroll = 8;
constexpr int kMaxTopk = 1024;

__device__ __forceinline__ unsigned long long composite(uint32_t key, int page) {
    return ((unsigned long long)key << 16) | (unsigned long long)(0xFFFFu - (unsigned)page);
}

template <typename T, int G>
__global__ void __launch_bounds__(kSelThreads, 2)
select_kernel(const T* __restrict__ q, const T* __restrict__ summaries, int64_t summary_stride,
              const int32_t* __restrict__ kv_indices, const int32_t* __restrict__ kv_indptr,
              const int32_t* __restrict__ kv_last_page_len, int topk, int key_cap,
              int32_t* __restrict__ out_pages, int32_t* __restrict__ out_logical,
              float* __restrict__ out_scores, int Hkv, int64_t num_pages, int32_t* status) {
    extern __shared__ uint32_t keys[];                 // one key per scored page
    __shared__ float qbar[kHeadDim];
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long sel[kMaxTopk];
    __shared__ int s_digit, s_greater, s_bincount, s_count;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hl = lane & 15;       // lane inside its 16-lane group
    const int grp = tid >> 4;       // 16-lane group inside the CTA
    const int64_t bh = blockIdx.x;
    const int b = (int)(bh / Hkv), h = (int)(bh % Hkv);
    const int stride_out = topk + 1;
    int32_t* row_pages = out_pages + bh * stride_out;
    int32_t* row_logical = out_logical ? out_logical + bh * stride_out : nullptr;

    const int beg = kv_indptr[b], end = kv_indptr[b + 1];
    const int n_pages = end - beg;
    const int last = (n_pages > 0) ? kv_last_page_len[b] : 1;
    const int n_scored = n_pages - 1;
    const bool bad = n_pages > 0 && (last < 1 || last > kPageSize || n_scored > summary_stride ||
                                     n_scored > key_cap);
    if (n_pages <= 0 || bad) {
        if (bad && tid == 0) report(status, KTK_STATUS_BAD_TABLE);
        for (int i = tid; i < stride_out; i += kSelThreads) {
            row_pages[i] = -1;
            if (row_logical) row_logical[i] = -1;
        }
        return;
    }

    const bool need_select = n_scored > topk;
    if (need_select || out_scores != nullptr) {
        if (tid < kHeadDim) {
            const T* qp = q + ((int64_t)b * Hkv * G + (int64_t)h * G) * kHeadDim + tid;
            float acc = 0.0f;
#pragma unroll
            for (int g = 0; g < G; ++g) acc = __fadd_rn(acc, to_f32(qp[g * kHeadDim]));
            qbar[tid] = __fmul_rn(acc, 1.0f / (float)G);
        }
        __syncthreads();
        float qr[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) qr[e] = qbar[8 * hl + e];

        const T* sbase = summaries + bh * summary_stride * kHeadDim + hl * 8;
        float* score_row = out_scores ? out_scores + bh * summary_stride : nullptr;
        constexpr int kRowsPerIt = kSelThreads / 16;
        for (int r0 = 0; r0 < n_scored; r0 += kRowsPerIt * kSelUnroll) {
            float x[kSelUnroll][8];
#pragma unroll
            for (int u = 0; u < kSelUnroll; ++u) {
                const int r = r0 + u * kRowsPerIt + grp;
                if (r < n_scored) {
                    load8(sbase + (int64_t)r * kHeadDim, x[u]);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[u][e] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < kSelUnroll; ++u) {
                const int r = r0 + u * kRowsPerIt + grp;
                float acc = 0.0f;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc = __fmaf_rn(qr[e], x[u][e], acc);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1)
                    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
                acc = __fadd_rn(acc, 0.0f);
                if (hl == 0 && r < n_scored) {
                    keys[r] = score_to_key(acc);
                    if (score_row) score_row[r] = acc;
                }
            }
        }
    }

    if (!need_select) {
        // every scored page is taken, in page order, then the page being filled
        for (int i = tid; i < stride_out; i += kSelThreads) {
            int logical = -1, phys = -1;
            if (i <= n_scored) {
                logical = i;
                phys = kv_indices[beg + i];
                if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
            }
            row_pages[i] = phys;
            if (row_logical) row_logical[i] = logical;
        }
        return;
    }

    // ---- radix select of the topk-th largest 48-bit composite, 8 bits per pass ----
    unsigned long long prefix = 0, mask = 0;
    int need = topk;
    if (tid == 0) s_count = 0;
    for (int shift = 40; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < n_scored; i += kSelThreads) {
            const unsigned long long c = composite(keys[i], i);
            if ((c & mask) == prefix) atomicAdd(&hist[(unsigned)(c >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns bins 255-8l .. 248-8l, walked from the largest digit down
            unsigned cnt[8];
            unsigned mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                cnt[j] = hist[255 - 8 * lane - j];
                mine += cnt[j];
            }
            unsigned incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            unsigned running = incl - mine;   // elements in strictly larger bins
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (running < (unsigned)need && (unsigned)need <= running + cnt[j]) {
                    s_digit = 255 - 8 * lane - j;
                    s_greater = (int)running;
                    s_bincount = (int)cnt[j];
                }
                running += cnt[j];
            }
        }
        __syncthreads();
        need -= s_greater;
        prefix |= (unsigned long long)s_digit << shift;
        mask |= 0xFFull << shift;
        if (s_bincount == need) break;   // the whole bin is taken: threshold found
    }

    // ---- gather the topk composites >= threshold, sort them descending ----
    int kp = 1;
    while (kp < topk) kp <<= 1;
    for (int i = tid; i < n_scored; i += kSelThreads) {
        const unsigned long long c = composite(keys[i], i);
        if ((c & mask) >= prefix) {
            const int pos = atomicAdd(&s_count, 1);
            if (pos < kMaxTopk) sel[pos] = c;
        }
    }
    for (int i = topk + tid; i < kp; i += kSelThreads) sel[i] = 0ull;
    __syncthreads();
    for (int k2 = 2; k2 <= kp; k2 <<= 1) {
        for (int j = k2 >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < kp; i += kSelThreads) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = sel[i], c = sel[ixj];
                    const bool desc = (i & k2) == 0;
                    if (desc ? (a < c) : (a > c)) { sel[i] = c; sel[ixj] = a; }
                }
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < stride_out; i += kSelThreads) {
        const int logical = (i < topk) ? (int)(0xFFFFu - (unsigned)(sel[i] & 0xFFFFull)) : n_pages - 1;
        const int phys = kv_indices[beg + logical];
        if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
        row_pages[i] = phys;
        if (row_logical) row_logical[i] = logical;
    }
}

template <typename T, int G>
static int select_launch(const void* q, const void* summaries, int64_t summary_stride,
                         const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, int topk, int32_t* out_pages,
                         int32_t* out_logical, float* out_scores, const ktk_shape* s,
                         int32_t* status, cudaStream_t st) {
    int key_cap = (int)(summary_stride < kMaxScoredPages ? summary_stride : kMaxScoredPages);
    const size_t smem = (size_t)key_cap * sizeof(uint32_t);
    auto kern = select_kernel<T, G>;
    if (smem > 40 * 1024) {
        KTK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                     "ktk_select");
    }
    const int64_t bh = (int64_t)s->batch * s->num_kv_heads;
    kern<<<(unsigned)bh, kSelThreads, smem, st>>>(
        (const T*)q, (const T*)summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
        topk, key_cap, out_pages, out_logical, out_scores, s->num_kv_heads, s->num_pages, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_select");
    return KTK_OK;
}

template <typename T, typename... A>
static int select_group(int G, A... a) {
    switch (G) {
        case 1: return select_launch<T, 1>(a...);
        case 2: return select_launch<T, 2>(a...);
        case 4: return select_launch<T, 4>(a...);
        default: return select_launch<T, 8>(a...);
    }
}

}  // namespace ktk

using namespace ktk;

extern "C" int ktk_select(const void* q, const void* summaries, int64_t summary_stride,
                          const int32_t* kv_indices, const int32_t* kv_indptr,
                          const int32_t* kv_last_page_len, int32_t topk, int32_t* out_pages,
                          int32_t* out_logical, float* out_scores, const ktk_shape* shape,
                          int32_t* status, void* stream) {
    int rc = check_shape(shape, "ktk_select");
    if (rc != KTK_OK) return rc;
    if (topk < 1 || topk > kMaxTopk) {
        set_error("ktk_select: topk %d outside [1, %d]", topk, kMaxTopk);
        return topk < 1 ? KTK_ERR_ARG : KTK_ERR_TOO_LARGE;
    }
    if (shape->batch == 0) return KTK_OK;
    if (!q || !summaries || !kv_indices || !kv_indptr || !kv_last_page_len || !out_pages) {
        set_error("ktk_select: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (summary_stride <= 0) {
        set_error("ktk_select: summary_stride must be positive");
        return KTK_ERR_ARG;
    }
    if ((int64_t)shape->batch * shape->num_kv_heads > 2147483647LL) {
        set_error("ktk_select: batch * num_kv_heads exceeds the grid limit");
        return KTK_ERR_TOO_LARGE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (shape->dtype == KTK_F32)
        return select_group<float>(shape->group_size, q, summaries, summary_stride, kv_indices,
                                   kv_indptr, kv_last_page_len, (int)topk, out_pages, out_logical,
                                   out_scores, shape, status, st);
    return select_group<__nv_bfloat16>(shape->group_size, q, summaries, summary_stride, kv_indices,
                                       kv_indptr, kv_last_page_len, (int)topk, out_pages,
                                       out_logical, out_scores, shape, status, st);
}
