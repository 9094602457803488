// Paged flash-decode attention, bf16 tensor-core variant with TMA-staged pages.
//
// One CTA per (sequence, kv head, split): four consumer warps plus one producer
// warp.  The producer walks the page list and, for every page, issues four TMA
// tile loads (K and V, each as two 16-row x 128-byte boxes, 128-byte swizzle)
// into an 8 KiB stage of a shared-memory ring; an mbarrier per stage counts the
// bytes in.  Stage i belongs to consumer warp i mod 4, which runs the whole page
// on the tensor cores in the transposed form, so that the 16 tokens of a page
// fill the M dimension and the (up to 8) query heads of the group the N dimension:
//     S^T[16 tok x 8 heads]  = K[16 x 128] . Q^T          8 x mma.m16n8k16
//     O^T[128 x 8 heads]    += V^T[128 x 16] . P^T        8 x mma.m16n8k16
// K fragments come from ldmatrix, V^T fragments from ldmatrix.trans, P^T from the
// S^T accumulators through movmatrix.  Softmax runs in base 2 with an online
// maximum per head; each warp keeps its own (m, l, O^T) and the four warps merge
// through shared memory at the end.  HBM traffic is exactly the listed pages.
#include "ktk_decode.cuh"
#include "ktk_pipeline.cuh"

namespace ktk {

constexpr int kMmaConsumers = 4;                       // consumer warps
constexpr int kMmaThreads = (kMmaConsumers + 1) * 32;  // + one producer warp
constexpr int kStageBytes = 2 * kPageSize * kHeadDim * 2;   // K + V of one page, bf16: 8 KiB
constexpr int kHalfTile = kPageSize * 128;                   // 16 rows x 128 B
// Ring depth.  A multiple of the consumer count, so that a stage is always drained by the same
// warp: that warp then sees every phase of the stage's barrier in turn.  (A warp that only
// saw every other phase could mistake the completion of phase k-1 for that of phase k+1 --
// an mbarrier wait only tells two consecutive phases apart.)
constexpr int kMmaStages = 8;
static_assert(kMmaStages % kMmaConsumers == 0, "a stage must belong to one consumer warp");

struct MmaParams {
    DecodeParams d;
    int G;
};

// byte offset of 16-byte chunk `c16` (0..15 across the 256-byte row) of token row `tok`
// inside a K or V tile stored as two 128-byte-swizzled half tiles
__device__ __forceinline__ uint32_t tile_off(int tok, int c16) {
    return (uint32_t)((c16 >> 3) * kHalfTile + tok * 128 + (((c16 & 7) ^ (tok & 7)) << 4));
}

__global__ void __launch_bounds__(kMmaThreads, 3)
decode_mma_kernel(const MmaParams p, const __grid_constant__ CUtensorMap kv_map) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMmaStages];
    __shared__ __align__(8) uint64_t empty_bar[kMmaStages];
    __shared__ int stage_tag[kMmaStages];     // issue index + 1 of the page in the stage, negated if skipped
    __shared__ int abort_flag;
    __shared__ int issued_total;
    __shared__ float red_m[kMmaConsumers][8], red_l[kMmaConsumers][8];

    // the swizzle pattern is a function of the shared-memory address: stages start on 1 KiB
    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const DecodeParams& d = p.d;
    const int G = p.G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = d.num_splits;
    const int64_t bh = blockIdx.x / S;
    const int split = blockIdx.x % S;
    const int b = (int)(bh / d.Hkv), h = (int)(bh % d.Hkv);
    const int Hq = d.Hkv * G;

    bool bad;
    const EntryList el = entry_list(d, b, h, bad);
    if (bad && tid == 0 && split == 0) report(d.status, KTK_STATUS_BAD_TABLE);
    const int per = (el.cnt + S - 1) / S;
    const int e0 = split * per;
    const int e1 = (e0 + per < el.cnt) ? e0 + per : el.cnt;
    const int n_entries = (e1 > e0) ? e1 - e0 : 0;

    if (tid == 0) {
        for (int s = 0; s < kMmaStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        abort_flag = 0;
        issued_total = 0;
        mbar_init_fence();
    }
    __syncthreads();

    const int gid = lane >> 2, tig = lane & 3;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // heads 2*tig and 2*tig+1
    float acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;

    if (warp == kMmaConsumers) {
        // ---------------- producer warp ----------------
        if (lane == 0) prefetch_tensormap(&kv_map);
        int issued = 0;
        int next_ids = (e0 + lane < e1) ? el.ptr[e0 + lane] : -1;
        bool alive = true;
        for (int base = e0; base < e1 && alive; base += 32) {
            const int ids = next_ids;
            next_ids = (base + 32 + lane < e1) ? el.ptr[base + 32 + lane] : -1;   // one chunk ahead
            const int chunk = (e1 - base < 32) ? e1 - base : 32;
            for (int j = 0; j < chunk && alive; ++j) {
                const int64_t page = __shfl_sync(0xffffffffu, ids, j);
                if (lane == 0) {
                    const int i = issued;
                    const int s = i % kMmaStages;
                    if (i >= kMmaStages && !mbar_wait(&empty_bar[s], ((i / kMmaStages) - 1) & 1, &abort_flag)) {
                        alive = false;
                    } else if (page < 0 || page >= d.num_pages) {
                        report(d.status, KTK_STATUS_BAD_PAGE);
                        stage_tag[s] = -(i + 1);
                        mbar_arrive(&full_bar[s]);          // nothing to load: release the consumer
                        issued = i + 1;
                    } else {
                        stage_tag[s] = i + 1;
                        uint8_t* dst = stages + s * kStageBytes;
                        const int y = (int)(page * (2 * kPageSize));      // token row of K slot 0
                        mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
                        tma_load_3d(dst, &kv_map, &full_bar[s], 0, h, y);
                        tma_load_3d(dst + kHalfTile, &kv_map, &full_bar[s], 64, h, y);
                        tma_load_3d(dst + 2 * kHalfTile, &kv_map, &full_bar[s], 0, h, y + kPageSize);
                        tma_load_3d(dst + 3 * kHalfTile, &kv_map, &full_bar[s], 64, h, y + kPageSize);
                        issued = i + 1;
                    }
                }
                alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
            }
        }
        if (lane == 0) issued_total = issued;
    } else {
        // ---------------- consumer warps ----------------
        // Q^T fragments: head gid, elements 16*ks + 2*tig (+8); heads past the group are zero
        uint32_t qb[8][2];
        {
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(
                (const __nv_bfloat16*)d.q + ((int64_t)b * Hq + (int64_t)h * G + gid) * kHeadDim);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qb[ks][0] = (gid < G) ? __ldg(qp + ks * 8 + tig) : 0u;
                qb[ks][1] = (gid < G) ? __ldg(qp + ks * 8 + 4 + tig) : 0u;
            }
        }
        const uint32_t stage_base = smem_u32(stages);
        // per-lane ldmatrix row addresses (relative to the tile): lane supplies row (lane & 7) of matrix lane >> 3
        const int mj = lane >> 3, mr = lane & 7;
        const int k_tok = mr + 8 * (mj & 1), k_c = mj >> 1;     // K:  matrices (tok 0-7 | 8-15) x (chunk 2ks | 2ks+1)
        const int v_tok = mr + 8 * (mj >> 1), v_c = mj & 1;     // V^T: matrices (chunk 2mt | 2mt+1) x (tok 0-7 | 8-15)

        for (int i = warp; i < n_entries; i += kMmaConsumers) {
            const int s = i % kMmaStages;
            // the vote keeps the warp together should a single lane give up
            if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i / kMmaStages) & 1, &abort_flag))) break;
            const int tag = stage_tag[s];
            if (tag != i + 1 && tag != -(i + 1)) {
                // the stage does not hold the page this warp is waiting for: stop rather than compute on it
                if (lane == 0) { report(d.status, KTK_STATUS_INTERNAL); abort_flag = 1; }
                break;
            }
            if (tag > 0) {
                const int e = e0 + i;
                const int ntok = entry_tokens(el, e);
                const uint32_t kt = stage_base + s * kStageBytes;
                const uint32_t vt = kt + 2 * kHalfTile;
                if (ntok < kPageSize) {
                    // rows past the fill level may hold anything: clear them in V so that 0 * x stays 0
                    uint8_t* vrow = stages + s * kStageBytes + 2 * kHalfTile;
                    for (int c = lane; c < (kPageSize - ntok) * 16; c += 32) {
                        const int t = ntok + (c >> 4), cc = c & 15;
                        *reinterpret_cast<uint4*>(vrow + (cc >> 3) * kHalfTile + t * 128 + ((cc & 7) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
                // S^T = K . Q^T, two accumulators to shorten the dependency chain
                float s_a[4] = {0.f, 0.f, 0.f, 0.f}, s_b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < 8; ks += 2) {
                    uint32_t ka[4], kb[4];
                    ldmatrix_x4(ka, kt + tile_off(k_tok, 2 * ks + k_c));
                    ldmatrix_x4(kb, kt + tile_off(k_tok, 2 * ks + 2 + k_c));
                    mma_bf16(s_a, ka, qb[ks][0], qb[ks][1]);
                    mma_bf16(s_b, kb, qb[ks + 1][0], qb[ks + 1][1]);
                }
                // scores of tokens gid and gid+8 for heads 2*tig, 2*tig+1 (log2 domain)
                float s00 = (s_a[0] + s_b[0]) * d.scale_log2, s01 = (s_a[1] + s_b[1]) * d.scale_log2;
                float s10 = (s_a[2] + s_b[2]) * d.scale_log2, s11 = (s_a[3] + s_b[3]) * d.scale_log2;
                if (gid >= ntok) { s00 = -INFINITY; s01 = -INFINITY; }
                if (gid + 8 >= ntok) { s10 = -INFINITY; s11 = -INFINITY; }
                float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
                }
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: token 0 is valid
                const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
                // probabilities, rounded to bf16 once so that the normaliser matches what multiplies V
                const uint32_t p_lo = pack_bf16(exp2f(s00 - mn0), exp2f(s01 - mn1));   // tokens 0-7
                const uint32_t p_hi = pack_bf16(exp2f(s10 - mn0), exp2f(s11 - mn1));   // tokens 8-15
                float sum0 = __uint_as_float(p_lo << 16) + __uint_as_float(p_hi << 16);
                float sum1 = __uint_as_float(p_lo & 0xffff0000u) + __uint_as_float(p_hi & 0xffff0000u);
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1) {
                    sum0 += __shfl_xor_sync(0xffffffffu, sum0, off);
                    sum1 += __shfl_xor_sync(0xffffffffu, sum1, off);
                }
                m0 = mn0; m1 = mn1;
                l0 = l0 * al0 + sum0;
                l1 = l1 * al1 + sum1;
                // P^T as the B operand: transpose the two 8x8 (token x head) blocks
                const uint32_t pb0 = movmatrix_trans(p_lo);
                const uint32_t pb1 = movmatrix_trans(p_hi);
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    uint32_t va[4];
                    ldmatrix_x4_trans(va, vt + tile_off(v_tok, 2 * mt + v_c));
                    acc[mt][0] *= al0; acc[mt][1] *= al1; acc[mt][2] *= al0; acc[mt][3] *= al1;
                    mma_bf16(acc[mt], va, pb0, pb1);
                }
                if (ntok < kPageSize) fence_proxy_async();   // the cleared rows were written by ordinary stores
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
    }

    __syncthreads();   // every page consumed (or the CTA gave up): stage memory is free
    if (abort_flag) {
        if (tid == 0) {
            report(d.status, KTK_STATUS_TIMEOUT);
            // wait, again bounded, for copies still in flight before the CTA's shared memory is released
            volatile int never = 0;
            const int total = issued_total;
            for (int i = (total > kMmaStages ? total - kMmaStages : 0); i < total; ++i)
                mbar_wait(&full_bar[i % kMmaStages], (i / kMmaStages) & 1, &never);
        }
        return;
    }

    // ---- merge the consumer warps (stage memory reused as the exchange buffer) ----
    float* red_o = reinterpret_cast<float*>(stages);          // [warp][head][128]
    if (warp < kMmaConsumers) {
        if (gid == 0) {
            red_m[warp][2 * tig] = m0; red_m[warp][2 * tig + 1] = m1;
            red_l[warp][2 * tig] = l0; red_l[warp][2 * tig + 1] = l1;
        }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            float* o0 = red_o + ((warp * 8 + 2 * tig) * kHeadDim) + 16 * mt + gid;
            o0[0] = acc[mt][0];
            o0[kHeadDim] = acc[mt][1];
            o0[8] = acc[mt][2];
            o0[kHeadDim + 8] = acc[mt][3];
        }
    }
    __syncthreads();
    if (tid < kHeadDim) {
        const int dd = tid;
        for (int g = 0; g < G; ++g) {
            float M = red_m[0][g];
#pragma unroll
            for (int w = 1; w < kMmaConsumers; ++w) M = fmaxf(M, red_m[w][g]);
            float L = 0.0f, O = 0.0f;
            if (M != -INFINITY) {
#pragma unroll
                for (int w = 0; w < kMmaConsumers; ++w) {
                    const float wt = exp2f(red_m[w][g] - M);
                    L += wt * red_l[w][g];
                    O += wt * red_o[(w * 8 + g) * kHeadDim + dd];
                }
            }
            const int64_t qh = (int64_t)b * Hq + (int64_t)h * G + g;
            if (S == 1) {
                ((__nv_bfloat16*)d.o)[qh * kHeadDim + dd] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
            } else {
                d.ws_o[(qh * S + split) * kHeadDim + dd] = O;
                if (dd == 0) {
                    d.ws_ml[(qh * S + split) * 2 + 0] = M;
                    d.ws_ml[(qh * S + split) * 2 + 1] = L;
                }
            }
        }
    }
}

int launch_decode_mma(const DecodeParams& p, int G, cudaStream_t st) {
    // tensor map over the cache seen as [token rows = pages*2*16][Hkv][128], innermost first
    CUtensorMap map;
    const uint64_t dims[3] = {(uint64_t)kHeadDim, (uint64_t)p.Hkv, (uint64_t)p.num_pages * 2 * kPageSize};
    const uint64_t strides[2] = {(uint64_t)kHeadDim * 2, (uint64_t)p.Hkv * kHeadDim * 2};
    const uint32_t box[3] = {64, 1, (uint32_t)kPageSize};
    if (dims[2] >= (1ull << 31)) {
        set_error("ktk decode: %lld pages exceed the tensor-core variant's 2^26-page limit", (long long)p.num_pages);
        return KTK_ERR_TOO_LARGE;
    }
    int rc = make_tensor_map_3d(&map, p.cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B, "ktk decode");
    if (rc != KTK_OK) return rc;
    const int smem = kMmaStages * kStageBytes + 1024;
    KTK_CUDA_TRY(cudaFuncSetAttribute(decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "ktk decode (mma)");
    MmaParams mp;
    mp.d = p;
    mp.G = G;
    const int64_t ctas = (int64_t)p.batch * p.Hkv * p.num_splits;
    decode_mma_kernel<<<(unsigned)ctas, kMmaThreads, smem, st>>>(mp, map);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk decode (mma)");
    return KTK_OK;
}

}  // namespace ktk
