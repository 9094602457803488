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
#include "ktk_decode_mma.cuh"

namespace ktk {

struct MmaParams {
    DecodeParams d;
    int G;
};

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
    MmaState ms;                                                   // heads 2*tig and 2*tig+1
    ms.reset();

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
                        tma_load_page(stages + s * kStageBytes, &kv_map, &full_bar[s], page, h);
                        issued = i + 1;
                    }
                }
                alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
            }
        }
        if (lane == 0) issued_total = issued;
    } else {
        // ---------------- consumer warps ----------------
        uint32_t qb[8][2];
        load_q_frags(qb, d.q, (int64_t)b * Hq + (int64_t)h * G, G, lane);

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
            if (tag > 0)
                mma_consume_page(ms, stages + s * kStageBytes, entry_tokens(el, e0 + i), qb, d.scale_log2, lane);
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
            red_m[warp][2 * tig] = ms.m0; red_m[warp][2 * tig + 1] = ms.m1;
            red_l[warp][2 * tig] = ms.l0; red_l[warp][2 * tig + 1] = ms.l1;
        }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            float* o0 = red_o + ((warp * 8 + 2 * tig) * kHeadDim) + 16 * mt + gid;
            o0[0] = ms.acc[mt][0];
            o0[kHeadDim] = ms.acc[mt][1];
            o0[8] = ms.acc[mt][2];
            o0[kHeadDim + 8] = ms.acc[mt][3];
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

int make_kv_tensor_map(CUtensorMap* map, const DecodeParams& p) {
    const uint64_t dims[3] = {(uint64_t)kHeadDim, (uint64_t)p.Hkv, (uint64_t)p.num_pages * 2 * kPageSize};
    const uint64_t strides[2] = {(uint64_t)kHeadDim * 2, (uint64_t)p.Hkv * kHeadDim * 2};
    const uint32_t box[3] = {64, 1, (uint32_t)kPageSize};
    if (dims[2] >= (1ull << 31)) {
        set_error("ktk decode: %lld pages exceed the tensor-core variant's 2^26-page limit", (long long)p.num_pages);
        return KTK_ERR_TOO_LARGE;
    }
    return make_tensor_map_3d(map, p.cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B, "ktk decode");
}

int launch_decode_mma(const DecodeParams& p, int G, cudaStream_t st) {
    CUtensorMap map;
    int rc = make_kv_tensor_map(&map, p);
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
