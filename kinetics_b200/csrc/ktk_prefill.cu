// Chunked causal prefill attention over the paged KV cache.
//
// The new tokens of every sequence (already written to their pages by ktk_append_tokens) attend the
// whole history of their sequence up to their own position.  Pages are read through the page table where
// they lie: no gathered copy of the history, no [new, total] mask; every sequence of the batch is served by
// one launch.  Replaces flashinfer.single_prefill_with_kv_cache(q, k_cache[:total], v_cache[:total],
// causal=True) of LiteSys/litesys/attention/batch_cache.py:129-145.
//
// bf16 (tensor cores): one CTA per (sequence, kv head, tile of 32 / G new tokens).  A producer warp walks
// the page list up to the tile's last position and stages each page (K and V, 8 KiB) with four TMA tile
// loads into a shared-memory ring; the four consumer warps all read every staged page, each for its own 8
// columns -- (token, head) pairs of the query group -- in the transposed form of the decode kernels:
//     S^T[16 keys x 8 columns] = K[16 x 128] . Q^T        8 x mma.m16n8k16
//     O^T[128 x 8 columns]    += V^T[128 x 16] . P^T      8 x mma.m16n8k16
// with a per-column horizon (keys behind the column's own token are masked).  A page is read once per 32
// columns, so a prompt of n tokens moves n / (32 / G) * pages * 8 KiB through L2 per kv head.
//
// fp32 (and bf16 on request): every new token becomes one row of the dense paged decode with its own
// page count and fill level (`prefill_rows_kernel` writes those three ints per row), which runs the fp32
// FMA decode kernel over the same page list.
#include "ktk_decode_mma.cuh"
#include "ktk_prefill_umma.cuh"

namespace ktk {

constexpr int kPfConsumers = 4;
constexpr int kPfThreads = (kPfConsumers + 1) * 32;
constexpr int kPfStages = 6;

struct PrefillParams {
    const void* q;
    void* o;
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

__global__ void __launch_bounds__(kPfThreads, 3)
prefill_mma_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap kv_map) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kPfStages];
    __shared__ __align__(8) uint64_t empty_bar[kPfStages];
    __shared__ int stage_tag[kPfStages];      // issue index + 1 of the page in the stage, negated if skipped
    __shared__ int abort_flag;
    __shared__ int issued_total;
    __shared__ float red_l[kPfConsumers][8];

    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z, h = blockIdx.y;
    const int G = p.G, Hq = p.Hkv * G;
    const int tpw = 8 / G;                          // new tokens per consumer warp (G = 1, 2, 4 or 8)
    const int tpc = tpw * kPfConsumers;             // ... per CTA
    const int q0 = p.q_indptr[b];
    const int n_new = p.q_indptr[b + 1] - q0;
    const int tok0 = blockIdx.x * tpc;
    if (tok0 >= n_new) return;                      // uniform for the CTA: nothing initialised yet

    const SeqPages sp = seq_pages(p.kv_indptr, p.page_count, p.kv_last_page_len, p.sink_tokens, b);
    const int base_pos = sp.total - n_new;          // position of the sequence's first new token
    if (sp.bad || base_pos < 0) {
        if (tid == 0) report(p.status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int tok_hi = (tok0 + tpc < n_new ? tok0 + tpc : n_new) - 1;
    int n_need, last_unused;
    pages_for(base_pos + tok_hi + 1, sp.first_fill, n_need, last_unused);
    if (n_need > sp.n_pages) n_need = sp.n_pages;

    if (tid == 0) {
        for (int s = 0; s < kPfStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kPfConsumers);
        }
        abort_flag = 0;
        issued_total = 0;
        mbar_init_fence();
    }
    __syncthreads();

    const int gid = lane >> 2, tig = lane & 3;
    MmaState ms;                                    // columns 2*tig and 2*tig+1 of this warp
    ms.reset();
    int vis0 = 0, vis1 = 0;                         // tokens those two columns may see (0: padding column)

    if (warp == kPfConsumers) {
        // ---------------- producer warp ----------------
        if (lane == 0) {
            prefetch_tensormap(&kv_map);
            int issued = 0;
            for (int e = 0; e < n_need; ++e) {
                const int64_t page = p.kv_indices[sp.start + e];
                const int s = e % kPfStages;
                if (e >= kPfStages && !mbar_wait(&empty_bar[s], ((e / kPfStages) - 1) & 1, &abort_flag)) break;
                if (page < 0 || page >= p.num_pages) {
                    report(p.status, KTK_STATUS_BAD_PAGE);
                    stage_tag[s] = -(e + 1);
                    mbar_arrive(&full_bar[s]);          // nothing to load: release the consumers
                } else {
                    stage_tag[s] = e + 1;
                    tma_load_page(stages + s * kStageBytes, &kv_map, &full_bar[s], page, h);
                }
                issued = e + 1;
            }
            issued_total = issued;
        }
    } else {
        // ---------------- consumer warps ----------------
        // column c of this warp = new token tok0 + warp * tpw + c / G, head c % G of the group
        const int wtok0 = tok0 + warp * tpw;
        auto col_visible = [&](int c) {
            const int t = wtok0 + c / G;
            return t < n_new ? base_pos + t + 1 : 0;
        };
        vis0 = col_visible(2 * tig);
        vis1 = col_visible(2 * tig + 1);
        int warp_vis = 0;                           // the farthest any column of this warp sees
        {
            const int t = wtok0 + tpw - 1 < n_new ? wtok0 + tpw - 1 : n_new - 1;
            warp_vis = t >= wtok0 ? base_pos + t + 1 : 0;
        }
        uint32_t qb[8][2];
        {
            const int t = wtok0 + gid / G;
            const bool on = t < n_new;
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(
                (const __nv_bfloat16*)p.q + ((int64_t)(q0 + (on ? t : 0)) * Hq + (int64_t)h * G + gid % G) * kHeadDim);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qb[ks][0] = on ? __ldg(qp + ks * 8 + tig) : 0u;
                qb[ks][1] = on ? __ldg(qp + ks * 8 + 4 + tig) : 0u;
            }
        }
        for (int e = 0; e < n_need; ++e) {
            const int s = e % kPfStages;
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (e / kPfStages) & 1, &abort_flag))) break;
            const int tag = stage_tag[s];
            if (tag != e + 1 && tag != -(e + 1)) {
                if (lane == 0) { report(p.status, KTK_STATUS_INTERNAL); abort_flag = 1; }
                break;
            }
            const int first = page_first_pos(e, sp.first_fill);
            if (tag > 0 && first < warp_vis) {
                const int ntok = (e == sp.n_pages - 1) ? sp.last_fill : (e == 0 ? sp.first_fill : kPageSize);
                int lim0 = vis0 - first, lim1 = vis1 - first;
                lim0 = lim0 < 0 ? 0 : (lim0 > ntok ? ntok : lim0);
                lim1 = lim1 < 0 ? 0 : (lim1 > ntok ? ntok : lim1);
                mma_consume_page_t<true>(ms, stages + s * kStageBytes, ntok, qb, p.scale_log2, lane, lim0, lim1);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
    }

    __syncthreads();   // every page consumed (or the CTA gave up): stage memory is free
    if (abort_flag) {
        if (tid == 0) {
            report(p.status, KTK_STATUS_TIMEOUT);
            volatile int never = 0;
            const int total = issued_total;
            for (int i = (total > kPfStages ? total - kPfStages : 0); i < total; ++i)
                mbar_wait(&full_bar[i % kPfStages], (i / kPfStages) & 1, &never);
        }
        return;
    }

    // ---- write the columns: transpose O^T through shared memory, normalise, store rows of 128 ----
    float* red_o = reinterpret_cast<float*>(stages);          // [warp][column][128]
    if (warp < kPfConsumers) {
        if (gid == 0) { red_l[warp][2 * tig] = ms.l0; red_l[warp][2 * tig + 1] = ms.l1; }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            float* o0 = red_o + ((warp * 8 + 2 * tig) * kHeadDim) + 16 * mt + gid;
            o0[0] = ms.acc[mt][0];
            o0[kHeadDim] = ms.acc[mt][1];
            o0[8] = ms.acc[mt][2];
            o0[kHeadDim + 8] = ms.acc[mt][3];
        }
        __syncwarp();
        const int wtok0 = tok0 + warp * tpw;
        for (int c = 0; c < 8; ++c) {
            const int t = wtok0 + c / G;
            if (t >= n_new) break;
            const float l = red_l[warp][c];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const float4 v = *reinterpret_cast<const float4*>(red_o + (warp * 8 + c) * kHeadDim + lane * 4);
            uint2 packed;
            packed.x = pack_bf16(v.x * inv, v.y * inv);
            packed.y = pack_bf16(v.z * inv, v.w * inv);
            __nv_bfloat16* dst = (__nv_bfloat16*)p.o + ((int64_t)(q0 + t) * Hq + (int64_t)h * G + c % G) * kHeadDim;
            *reinterpret_cast<uint2*>(dst + lane * 4) = packed;
        }
    }
}

// One decode row per new token: where its page list starts, how many pages it sees, how many tokens of
// the last of them.  rows = [3][total_new]: start, count, last.
__global__ void prefill_rows_kernel(const int32_t* q_indptr, const int32_t* kv_indptr, const int32_t* page_count,
                                    const int32_t* kv_last_page_len, int sink, int batch, int64_t total_new,
                                    int32_t* rows, int32_t* status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_new) return;
    int lo = 0, hi = batch;                         // the sequence whose range [q_indptr[b], q_indptr[b+1]) holds i
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((int64_t)q_indptr[mid] <= i) lo = mid; else hi = mid;
    }
    const int b = lo;
    const SeqPages sp = seq_pages(kv_indptr, page_count, kv_last_page_len, sink, b);
    const int n_new = q_indptr[b + 1] - q_indptr[b];
    const int pos = sp.total - n_new + (int)(i - q_indptr[b]);
    int count = 0, last = 1;
    if (sp.bad || pos < 0 || i >= (int64_t)q_indptr[b + 1]) {
        report(status, KTK_STATUS_BAD_TABLE);
    } else {
        pages_for(pos + 1, sp.first_fill, count, last);
    }
    rows[i] = sp.start;
    rows[total_new + i] = count;
    rows[2 * total_new + i] = last;
}

static int launch_prefill_mma(const PrefillParams& p, const void* cache, int max_new_tokens, cudaStream_t st) {
    DecodeParams d{};                               // only what the tensor map needs
    d.cache = cache; d.Hkv = p.Hkv; d.num_pages = p.num_pages;
    CUtensorMap map;
    int rc = make_kv_tensor_map(&map, d);
    if (rc != KTK_OK) return rc;
    const int smem = kPfStages * kStageBytes + 1024;
    KTK_CUDA_TRY(cudaFuncSetAttribute(prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "ktk_prefill_attention");
    const int tpc = (8 / p.G) * kPfConsumers;
    const dim3 grid((unsigned)((max_new_tokens + tpc - 1) / tpc), (unsigned)p.Hkv, (unsigned)p.batch);
    prefill_mma_kernel<<<grid, kPfThreads, smem, st>>>(p, map);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_prefill_attention");
    return KTK_OK;
}

}  // namespace ktk

using namespace ktk;

extern "C" size_t ktk_prefill_workspace_bytes(int64_t total_new_tokens, int32_t dtype, int32_t variant) {
    if (total_new_tokens <= 0) return 0;
    const bool rows_path = dtype != KTK_BF16 || variant == KTK_VARIANT_SIMT;
    return rows_path ? (size_t)total_new_tokens * 3 * sizeof(int32_t) : 0;
}

extern "C" int ktk_prefill_attention(const void* q, const int32_t* q_indptr, int64_t total_new_tokens,
                                     int32_t max_new_tokens, const void* kv_cache, const int32_t* kv_indices,
                                     const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                     const ktk_view* view_in, float sm_scale, void* o, void* workspace,
                                     size_t workspace_bytes, int32_t variant, const ktk_shape* s, int32_t* status,
                                     void* stream) {
    const char* who = "ktk_prefill_attention";
    int rc = check_shape(s, who);
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, who);
    if (rc != KTK_OK) return rc;
    if (s->batch == 0 || total_new_tokens == 0) return KTK_OK;
    if (!q || !q_indptr || !kv_cache || !kv_indices || !kv_indptr || !kv_last_page_len || !o || total_new_tokens < 0 ||
        max_new_tokens < 1) {
        set_error("%s: null pointer or negative size", who);
        return KTK_ERR_ARG;
    }
    if (variant != KTK_VARIANT_AUTO && variant != KTK_VARIANT_SIMT && variant != KTK_VARIANT_MMA &&
        variant != KTK_VARIANT_UMMA) {
        set_error("%s: unknown variant %d", who, variant);
        return KTK_ERR_ARG;
    }
    const int G = s->group_size;
    const bool mma_ok = s->dtype == KTK_BF16 && (G == 1 || G == 2 || G == 4 || G == 8);
    if ((variant == KTK_VARIANT_MMA || variant == KTK_VARIANT_UMMA) && !mma_ok) {
        set_error("%s: the tensor-core variant needs bf16 and a group size of 1, 2, 4 or 8", who);
        return KTK_ERR_UNSUPPORTED;
    }
    const View view = make_view(view_in);
    cudaStream_t st = (cudaStream_t)stream;
    if (variant != KTK_VARIANT_SIMT && mma_ok) {
        if (s->batch > 65535 || s->num_kv_heads > 65535) {
            set_error("%s: more than 65535 sequences or kv heads in one launch", who);
            return KTK_ERR_TOO_LARGE;
        }
        if (variant != KTK_VARIANT_MMA) {             // KTK_VARIANT_AUTO and KTK_VARIANT_UMMA: the tcgen05 kernel
            PrefillUmmaParams u;
            u.q = q; u.o = o; u.cache = kv_cache; u.q_indptr = q_indptr; u.kv_indices = kv_indices;
            u.kv_indptr = kv_indptr; u.kv_last_page_len = kv_last_page_len; u.page_count = view.page_count;
            u.sink_tokens = view.sink_tokens; u.batch = s->batch; u.Hkv = s->num_kv_heads; u.G = G;
            u.num_pages = s->num_pages; u.scale_log2 = sm_scale * kLog2e; u.status = status;
            return launch_prefill_umma(u, max_new_tokens, st);
        }
        PrefillParams p;
        p.q = q; p.o = o; p.q_indptr = q_indptr; p.kv_indices = kv_indices; p.kv_indptr = kv_indptr;
        p.kv_last_page_len = kv_last_page_len; p.page_count = view.page_count; p.sink_tokens = view.sink_tokens;
        p.batch = s->batch; p.Hkv = s->num_kv_heads; p.G = G; p.num_pages = s->num_pages;
        p.scale_log2 = sm_scale * kLog2e; p.status = status;
        return launch_prefill_mma(p, kv_cache, max_new_tokens, st);
    }
    // every new token as a row of the dense paged decode
    const size_t need = ktk_prefill_workspace_bytes(total_new_tokens, s->dtype, KTK_VARIANT_SIMT);
    if (workspace == nullptr || workspace_bytes < need) {
        set_error("%s: workspace of %zu bytes needed (ktk_prefill_workspace_bytes), got %zu", who, need,
                  workspace ? workspace_bytes : (size_t)0);
        return KTK_ERR_WORKSPACE;
    }
    if (total_new_tokens > 2147483647LL / (s->num_kv_heads > 0 ? s->num_kv_heads : 1)) {
        set_error("%s: too many new tokens for one launch", who);
        return KTK_ERR_TOO_LARGE;
    }
    int32_t* rows = (int32_t*)workspace;
    const int threads = 128;
    prefill_rows_kernel<<<(unsigned)((total_new_tokens + threads - 1) / threads), threads, 0, st>>>(
        q_indptr, kv_indptr, view.page_count, kv_last_page_len, view.sink_tokens, s->batch, total_new_tokens, rows,
        status);
    KTK_CUDA_TRY(cudaGetLastError(), who);
    DecodeParams d{};
    d.q = q; d.cache = kv_cache; d.o = o; d.entries = kv_indices;
    d.kv_indptr = rows; d.page_count = rows + total_new_tokens; d.kv_last_page_len = rows + 2 * total_new_tokens;
    d.topk = -1; d.entry_stride = 0; d.batch = (int)total_new_tokens; d.Hkv = s->num_kv_heads;
    d.num_pages = s->num_pages; d.scale_log2 = sm_scale * kLog2e; d.num_splits = 1;
    d.ws_ml = nullptr; d.ws_o = nullptr; d.status = status;
    d.sink_tokens = view.sink_tokens; d.local_tokens = view.local_tokens;
    return launch_decode_simt(d, s->dtype, G, st);
}
