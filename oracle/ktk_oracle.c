/*
 * CPU oracle for block top-k paged decode attention -- TEST INFRASTRUCTURE ONLY.
 *
 * Plain C restatement of the algorithm of Infini-AI-Lab/Kinetics for this path.
 * It is the checker the CUDA kernels are compared with (and the timed CPU
 * baseline of the benchmark); nothing in the product path may call it.
 *
 * Parity pin: the reference ships no tests or golden vectors.  This restatement
 * is pinned against the reference's own Python functions run on CPU
 * (LiteSys/litesys/attention/sparsity_utils.py blockwise_topk_sparsity and the
 * Triton kernels of cache_utils.py under the Triton interpreter); the vectors
 * they produced are stored under tests/golden/ with the script that made them.
 *
 * What each function follows (file:line inside the reference project):
 *   ktko_summaries   mean key of a 16-token block: sparsity_utils.py:37 (block mean,
 *                    moved in front of the dot product by linearity); replaces the
 *                    random compressed_key_cache of benchmark/blocktopk_decoder.py:166-168
 *   ktko_scores      benchmark/blocktopk_decoder.py:216 (einsum over d, mean over the
 *                    query group), grouping per kv head as sparsity_utils.py:36
 *   ktko_select      benchmark/blocktopk_decoder.py:217-221 (top-k, logical->physical,
 *                    always-on last page); dense when few pages: sparsity_utils.py:27-32
 *   ktko_decode      mylib::decode = flashinfer paged decode, benchmark/blocktopk_decoder.py:176-178;
 *                    the same math as cache_utils.py:86 (scaled dot), :116-130 (softmax), :165 (sum p.V)
 *   ktko_append      flashinfer.append_paged_kv_cache, benchmark/blocktopk_decoder.py:38-46;
 *                    LiteSys copy_to_cache, cache_utils.py:5-51
 *
 * Layouts are those of include/ktk.h.  dtype: 0 = fp32, 1 = bf16 (uint16 storage).
 * The summation order of a score is fixed (see ktko_scores): the GPU kernel uses
 * the same order, so selected pages can be compared bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define D 128
#define P 16

static inline float bf16_to_f32(uint16_t x) {
    uint32_t u = (uint32_t)x << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round to nearest even, NaN kept quiet */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float ld(const void* base, int dtype, int64_t i) {
    return dtype == 0 ? ((const float*)base)[i] : bf16_to_f32(((const uint16_t*)base)[i]);
}
static inline void st(void* base, int dtype, int64_t i, float v) {
    if (dtype == 0) ((float*)base)[i] = v; else ((uint16_t*)base)[i] = f32_to_bf16(v);
}

static inline uint32_t score_key(float s) {
    s = s + 0.0f;
    uint32_t u;
    memcpy(&u, &s, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/* element index of K (kv=0) or V (kv=1) row `t` of head `h` in physical page `page` */
static inline int64_t kv_row(int64_t page, int kv, int t, int h, int Hkv) {
    return (((page * 2 + kv) * P + t) * (int64_t)Hkv + h) * D;
}

/* ---- append one token per sequence, optionally refreshing the last page's summary ---- */
int ktko_append(const void* k, const void* v, void* cache, void* summaries, int64_t summary_stride,
                const int32_t* kv_indices, const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                int B, int Hkv, int dtype) {
    for (int b = 0; b < B; ++b) {
        const int beg = kv_indptr[b], end = kv_indptr[b + 1];
        if (end - beg <= 0) continue;
        const int last = kv_last_page_len[b];
        const int64_t page = kv_indices[end - 1];
        for (int h = 0; h < Hkv; ++h) {
            for (int d = 0; d < D; ++d) {
                const int64_t src = ((int64_t)b * Hkv + h) * D + d;
                st(cache, dtype, kv_row(page, 0, last - 1, h, Hkv) + d, ld(k, dtype, src));
                st(cache, dtype, kv_row(page, 1, last - 1, h, Hkv) + d, ld(v, dtype, src));
            }
            if (summaries) {
                for (int d = 0; d < D; ++d) {
                    float acc = 0.0f;
                    for (int t = 0; t < last; ++t) acc = acc + ld(cache, dtype, kv_row(page, 0, t, h, Hkv) + d);
                    st(summaries, dtype, (((int64_t)b * Hkv + h) * summary_stride + (end - beg - 1)) * D + d,
                       acc / (float)last);
                }
            }
        }
    }
    return 0;
}

/* ---- summary of every page: fp32 sum over the filled slots in slot order, / count ---- */
int ktko_summaries(const void* cache, void* summaries, int64_t summary_stride, const int32_t* kv_indices,
                   const int32_t* kv_indptr, const int32_t* kv_last_page_len, int B, int Hkv, int dtype) {
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < B; ++b) {
        const int beg = kv_indptr[b], n_pages = kv_indptr[b + 1] - beg;
        for (int p = 0; p < n_pages; ++p) {
            const int c = (p == n_pages - 1) ? kv_last_page_len[b] : P;
            const int64_t page = kv_indices[beg + p];
            for (int h = 0; h < Hkv; ++h)
                for (int d = 0; d < D; ++d) {
                    float acc = 0.0f;
                    for (int t = 0; t < c; ++t) acc = acc + ld(cache, dtype, kv_row(page, 0, t, h, Hkv) + d);
                    st(summaries, dtype, (((int64_t)b * Hkv + h) * summary_stride + p) * D + d, acc / (float)c);
                }
        }
    }
    return 0;
}

/*
 * score[b,h,p] for the scored pages p < n_pages-1, in the contract's order:
 *   qbar[d] = (q[g=0][d] + ... + q[G-1][d]) * (1/G)
 *   part_j  = fma chain over elements 8j .. 8j+7 (j = 0..15), starting from 0
 *   tree    : part_j += part_(j^8); then ^4; ^2; ^1        (butterfly, all 16 lanes)
 *   score   = part_0 + 0.0f
 * scores: [B, Hkv, summary_stride] fp32 (entries past the scored pages untouched)
 */
int ktko_scores(const void* q, const void* summaries, int64_t summary_stride, const int32_t* kv_indptr,
                float* scores, int B, int Hkv, int G, int dtype) {
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv, h = bh % Hkv;
        const int n_scored = kv_indptr[b + 1] - kv_indptr[b] - 1;
        float qbar[D];
        const float inv_g = 1.0f / (float)G;
        for (int d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int g = 0; g < G; ++g) acc = acc + ld(q, dtype, (((int64_t)b * Hkv + h) * G + g) * D + d);
            qbar[d] = acc * inv_g;
        }
        for (int p = 0; p < n_scored; ++p) {
            const int64_t base = ((int64_t)bh * summary_stride + p) * D;
            float part[16];
            for (int j = 0; j < 16; ++j) {
                float acc = 0.0f;
                for (int e = 0; e < 8; ++e) acc = fmaf(qbar[8 * j + e], ld(summaries, dtype, base + 8 * j + e), acc);
                part[j] = acc;
            }
            for (int off = 8; off > 0; off >>= 1) {
                float nxt[16];
                for (int j = 0; j < 16; ++j) nxt[j] = part[j] + part[j ^ off];
                memcpy(part, nxt, sizeof(part));
            }
            scores[(int64_t)bh * summary_stride + p] = part[0] + 0.0f;
        }
    }
    return 0;
}

typedef struct { uint32_t key; int32_t page; } keyed;

/* larger key first, equal keys: lower page first */
static int keyed_cmp(const void* a, const void* b) {
    const keyed* x = (const keyed*)a;
    const keyed* y = (const keyed*)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    return x->page < y->page ? -1 : (x->page > y->page ? 1 : 0);
}

/*
 * Selection from scores.  out_logical / out_pages: [B, Hkv, topk+1], unused tail = -1.
 */
int ktko_select(const float* scores, int64_t summary_stride, const int32_t* kv_indices,
                const int32_t* kv_indptr, int topk, int32_t* out_pages, int32_t* out_logical, int B, int Hkv) {
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv;
        const int beg = kv_indptr[b], n_pages = kv_indptr[b + 1] - beg;
        int32_t* lo = out_logical + (int64_t)bh * (topk + 1);
        int32_t* ph = out_pages + (int64_t)bh * (topk + 1);
        for (int i = 0; i <= topk; ++i) { lo[i] = -1; ph[i] = -1; }
        if (n_pages <= 0) continue;
        const int n_scored = n_pages - 1;
        int cnt = 0;
        if (n_scored <= topk) {
            for (int p = 0; p < n_scored; ++p) lo[cnt++] = p;
        } else {
            keyed* ks = (keyed*)malloc(sizeof(keyed) * (size_t)n_scored);
            for (int p = 0; p < n_scored; ++p) {
                ks[p].key = score_key(scores[(int64_t)bh * summary_stride + p]);
                ks[p].page = p;
            }
            qsort(ks, (size_t)n_scored, sizeof(keyed), keyed_cmp);
            for (int i = 0; i < topk; ++i) lo[cnt++] = ks[i].page;
            free(ks);
        }
        lo[cnt++] = n_pages - 1;
        for (int i = 0; i < cnt; ++i) ph[i] = kv_indices[beg + lo[i]];
    }
    return 0;
}

/*
 * Attention over a page list, double precision throughout (the tolerance reference).
 * entries: sparse (topk >= 1): [B, Hkv, topk+1] physical pages; dense (topk < 0): kv_indices.
 * out: [B, Hq, D] fp32.
 */
int ktko_decode(const void* q, const void* cache, const int32_t* entries, int topk, const int32_t* kv_indptr,
                const int32_t* kv_last_page_len, float sm_scale, float* out, int B, int Hkv, int G, int dtype) {
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv, h = bh % Hkv;
        const int beg = kv_indptr[b], n_pages = kv_indptr[b + 1] - beg;
        float* ob = out + ((int64_t)bh * G) * D;
        for (int i = 0; i < G * D; ++i) ob[i] = 0.0f;
        if (n_pages <= 0) continue;
        const int32_t* list;
        int cnt;
        if (topk >= 0) {
            const int scored = n_pages - 1;
            cnt = (scored < topk ? scored : topk) + 1;
            list = entries + (int64_t)bh * (topk + 1);
        } else {
            cnt = n_pages;
            list = entries + beg;
        }
        const int last = kv_last_page_len[b];
        const int ntot = (cnt - 1) * P + last;
        double* logit = (double*)malloc(sizeof(double) * (size_t)ntot);
        for (int g = 0; g < G; ++g) {
            const int64_t qoff = ((int64_t)bh * G + g) * D;
            double mx = -INFINITY;
            for (int e = 0; e < cnt; ++e) {
                const int nt = (e == cnt - 1) ? last : P;
                for (int t = 0; t < nt; ++t) {
                    const int64_t kr = kv_row(list[e], 0, t, h, Hkv);
                    double acc = 0.0;
                    for (int d = 0; d < D; ++d) acc += (double)ld(q, dtype, qoff + d) * (double)ld(cache, dtype, kr + d);
                    acc *= (double)sm_scale;
                    logit[e * P + t] = acc;
                    if (acc > mx) mx = acc;
                }
            }
            double den = 0.0;
            double o[D];
            for (int d = 0; d < D; ++d) o[d] = 0.0;
            for (int e = 0; e < cnt; ++e) {
                const int nt = (e == cnt - 1) ? last : P;
                for (int t = 0; t < nt; ++t) {
                    const double w = exp(logit[e * P + t] - mx);
                    den += w;
                    const int64_t vr = kv_row(list[e], 1, t, h, Hkv);
                    for (int d = 0; d < D; ++d) o[d] += w * (double)ld(cache, dtype, vr + d);
                }
            }
            for (int d = 0; d < D; ++d) ob[g * D + d] = (float)(o[d] / den);
        }
        free(logit);
    }
    return 0;
}


/* ------------------------------------------------------------------------------------------
 * The same operations under a page view (sink_tokens, local_tokens) -- the LiteSys semantics of
 * LiteSys/litesys/attention/sparsity_utils.py:24-47: logical page 0 holds the `sink` first tokens
 * (sparsity_utils.py:24 `sink=4`), 16-token blocks are counted from the end of the sink (:33-37),
 * the blocks whose tokens all lie more than `local` tokens behind the end are scored
 * (`_n_dynamic`, :33), everything after them is always kept (`_local`, :34), and nothing is
 * dropped while `_n_dynamic / 16 <= topk` (:27-32).  sink = 0, local = 1 is the benchmark view.
 * ------------------------------------------------------------------------------------------ */
typedef struct { int n_pages, front, n_dyn, back, last; } page_split_t;

static page_split_t page_split(const int32_t* kv_indptr, const int32_t* kv_last_page_len, int b, int sink, int local) {
    page_split_t ps;
    ps.n_pages = kv_indptr[b + 1] - kv_indptr[b];
    ps.last = ps.n_pages > 0 ? kv_last_page_len[b] : P;
    ps.front = (sink > 0 && ps.n_pages > 0) ? 1 : 0;
    const int n_after = ps.n_pages - ps.front;
    const int len_after = n_after > 0 ? (n_after - 1) * P + ps.last : 0;
    const int dyn = len_after - local;
    ps.n_dyn = dyn > 0 ? dyn / P : 0;
    ps.back = n_after - ps.n_dyn;
    return ps;
}

static int page_tokens(const page_split_t* ps, int logical, int sink) {
    if (logical == ps->n_pages - 1) return ps->last;
    if (logical == 0 && ps->front) return sink;
    return P;
}

int ktko_summaries_v(const void* cache, void* summaries, int64_t summary_stride, const int32_t* kv_indices,
                     const int32_t* kv_indptr, const int32_t* kv_last_page_len, int sink, int B, int Hkv, int dtype) {
    for (int b = 0; b < B; ++b) {
        const page_split_t ps = page_split(kv_indptr, kv_last_page_len, b, sink, 1);
        const int beg = kv_indptr[b];
        for (int p = 0; p < ps.n_pages; ++p) {
            const int c = page_tokens(&ps, p, sink);
            const int64_t page = kv_indices[beg + p];
            for (int h = 0; h < Hkv; ++h)
                for (int d = 0; d < D; ++d) {
                    float acc = 0.0f;
                    for (int t = 0; t < c; ++t) acc = acc + ld(cache, dtype, kv_row(page, 0, t, h, Hkv) + d);
                    st(summaries, dtype, (((int64_t)b * Hkv + h) * summary_stride + p) * D + d, acc / (float)c);
                }
        }
    }
    return 0;
}

/* scores[b, h, logical page] for the scored pages front .. front + n_dyn - 1, same arithmetic as ktko_scores */
int ktko_scores_v(const void* q, const void* summaries, int64_t summary_stride, const int32_t* kv_indptr,
                  const int32_t* kv_last_page_len, int sink, int local, float* scores, int B, int Hkv, int G,
                  int dtype) {
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv, h = bh % Hkv;
        const page_split_t ps = page_split(kv_indptr, kv_last_page_len, b, sink, local);
        float qbar[D];
        const float inv_g = 1.0f / (float)G;
        for (int d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int g = 0; g < G; ++g) acc = acc + ld(q, dtype, (((int64_t)b * Hkv + h) * G + g) * D + d);
            qbar[d] = acc * inv_g;
        }
        for (int r = 0; r < ps.n_dyn; ++r) {
            const int64_t base = ((int64_t)bh * summary_stride + ps.front + r) * D;
            float part[16];
            for (int j = 0; j < 16; ++j) {
                float acc = 0.0f;
                for (int e = 0; e < 8; ++e) acc = fmaf(qbar[8 * j + e], ld(summaries, dtype, base + 8 * j + e), acc);
                part[j] = acc;
            }
            for (int off = 8; off > 0; off >>= 1) {
                float nxt[16];
                for (int j = 0; j < 16; ++j) nxt[j] = part[j] + part[j ^ off];
                memcpy(part, nxt, sizeof(part));
            }
            scores[(int64_t)bh * summary_stride + ps.front + r] = part[0] + 0.0f;
        }
    }
    return 0;
}

/* rows of `row_width` ints: [sink page][picks, best first, ties to the lowest page][tail pages], then -1 */
int ktko_select_v(const float* scores, int64_t summary_stride, const int32_t* kv_indices, const int32_t* kv_indptr,
                  const int32_t* kv_last_page_len, int topk, int sink, int local, int row_width,
                  int32_t* out_pages, int32_t* out_logical, int B, int Hkv) {
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv;
        const int beg = kv_indptr[b];
        const page_split_t ps = page_split(kv_indptr, kv_last_page_len, b, sink, local);
        int32_t* lo = out_logical + (int64_t)bh * row_width;
        int32_t* ph = out_pages + (int64_t)bh * row_width;
        for (int i = 0; i < row_width; ++i) { lo[i] = -1; ph[i] = -1; }
        if (ps.n_pages <= 0) continue;
        int cnt = 0;
        if (ps.n_dyn <= topk) {
            for (int p = 0; p < ps.n_pages; ++p) lo[cnt++] = p;
        } else {
            if (ps.front) lo[cnt++] = 0;
            keyed* ks = (keyed*)malloc(sizeof(keyed) * (size_t)ps.n_dyn);
            for (int r = 0; r < ps.n_dyn; ++r) {
                ks[r].key = score_key(scores[(int64_t)bh * summary_stride + ps.front + r]);
                ks[r].page = r;
            }
            qsort(ks, (size_t)ps.n_dyn, sizeof(keyed), keyed_cmp);
            for (int i = 0; i < topk; ++i) lo[cnt++] = ps.front + ks[i].page;
            free(ks);
            for (int p = ps.front + ps.n_dyn; p < ps.n_pages; ++p) lo[cnt++] = p;
        }
        for (int i = 0; i < cnt; ++i) ph[i] = kv_indices[beg + lo[i]];
    }
    return 0;
}

/* attention over the listed pages (sparse: rows of row_width; dense: topk < 0, entries = kv_indices) */
int ktko_decode_v(const void* q, const void* cache, const int32_t* entries, int topk, int sink, int local,
                  int row_width, const int32_t* kv_indptr, const int32_t* kv_last_page_len, float sm_scale,
                  float* out, int B, int Hkv, int G, int dtype) {
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * Hkv; ++bh) {
        const int b = bh / Hkv, h = bh % Hkv;
        const page_split_t ps = page_split(kv_indptr, kv_last_page_len, b, sink, local);
        float* ob = out + ((int64_t)bh * G) * D;
        for (int i = 0; i < G * D; ++i) ob[i] = 0.0f;
        if (ps.n_pages <= 0) continue;
        const int32_t* list;
        int cnt;
        if (topk >= 0) {
            cnt = ps.front + (ps.n_dyn < topk ? ps.n_dyn : topk) + ps.back;
            list = entries + (int64_t)bh * row_width;
        } else {
            cnt = ps.n_pages;
            list = entries + kv_indptr[b];
        }
        double* logit = (double*)malloc(sizeof(double) * (size_t)cnt * P);
        for (int g = 0; g < G; ++g) {
            const int64_t qoff = ((int64_t)bh * G + g) * D;
            double mx = -INFINITY;
            for (int e = 0; e < cnt; ++e) {
                const int nt = (e == cnt - 1) ? ps.last : ((e == 0 && ps.front) ? sink : P);
                for (int t = 0; t < nt; ++t) {
                    const int64_t kr = kv_row(list[e], 0, t, h, Hkv);
                    double acc = 0.0;
                    for (int d = 0; d < D; ++d) acc += (double)ld(q, dtype, qoff + d) * (double)ld(cache, dtype, kr + d);
                    acc *= (double)sm_scale;
                    logit[e * P + t] = acc;
                    if (acc > mx) mx = acc;
                }
            }
            double den = 0.0;
            double o[D];
            for (int d = 0; d < D; ++d) o[d] = 0.0;
            for (int e = 0; e < cnt; ++e) {
                const int nt = (e == cnt - 1) ? ps.last : ((e == 0 && ps.front) ? sink : P);
                for (int t = 0; t < nt; ++t) {
                    const double w = exp(logit[e * P + t] - mx);
                    den += w;
                    const int64_t vr = kv_row(list[e], 1, t, h, Hkv);
                    for (int d = 0; d < D; ++d) o[d] += w * (double)ld(cache, dtype, vr + d);
                }
            }
            for (int d = 0; d < D; ++d) ob[g * D + d] = (float)(o[d] / den);
        }
        free(logit);
    }
    return 0;
}


/* several tokens per sequence: k, v [total, Hkv, D] packed by sequence, append_indptr [B+1]
 * (the kv_append_indptr of flashinfer.append_paged_kv_cache, benchmark/blocktopk_decoder.py:38-46);
 * the page table describes the state after the append.  Summaries are not touched here. */
int ktko_append_tokens(const void* k, const void* v, const int32_t* append_indptr, void* cache,
                       const int32_t* kv_indices, const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                       int sink, int B, int Hkv, int dtype) {
    for (int b = 0; b < B; ++b) {
        const int a0 = append_indptr[b], n_app = append_indptr[b + 1] - a0;
        const int beg = kv_indptr[b], n_pages = kv_indptr[b + 1] - beg;
        if (n_app <= 0 || n_pages <= 0) continue;
        const int last = kv_last_page_len[b];
        const int len = sink == 0 ? (n_pages - 1) * P + last : (n_pages == 1 ? last : sink + (n_pages - 2) * P + last);
        for (int i = 0; i < n_app; ++i) {
            const int pos = len - n_app + i;
            const int lp = sink == 0 ? pos / P : (pos < sink ? 0 : 1 + (pos - sink) / P);
            const int sl = sink == 0 ? pos % P : (pos < sink ? pos : (pos - sink) % P);
            const int64_t page = kv_indices[beg + lp];
            for (int h = 0; h < Hkv; ++h)
                for (int d = 0; d < D; ++d) {
                    const int64_t src = (((int64_t)(a0 + i)) * Hkv + h) * D + d;
                    st(cache, dtype, kv_row(page, 0, sl, h, Hkv) + d, ld(k, dtype, src));
                    st(cache, dtype, kv_row(page, 1, sl, h, Hkv) + d, ld(v, dtype, src));
                }
        }
    }
    return 0;
}
