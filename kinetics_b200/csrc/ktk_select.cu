// GQA query x page-summary scoring fused with per-(sequence, kv head) top-k
// page selection.  HBM-bound: one streaming pass over the sequence's summaries
// (n_scored * D elements), everything else stays in shared memory.
//
// The arithmetic order of a score is part of the contract (selection must be
// bit-exact against the CPU oracle):
//   qbar[d]  = (q[g=0][d] + q[1][d] + ... + q[G-1][d]) * (1/G)      fp32, in g order
//   sixteen chains over the 8-element chunks j = 0..15 of the summary row:
//   part_j   = fma(qbar[8j+7], s[8j+7], ... fma(qbar[8j], s[8j], 0))   in element order
//   then four butterfly levels part_j += part_(j xor off), off = 8, 4, 2, 1
//   score    = part_0 + 0.0f
// The kernel gives the chains j, j+4, j+8, j+12 to one lane (four lanes per row): the levels
// "xor 8" and "xor 4" are then adds inside the lane, "xor 2" and "xor 1" two shuffles; fp32
// addition is commutative, so the bits are those of the sixteen-lane butterfly.
// Selection orders pages by the 48-bit composite (key(score) << 16) | (0xFFFF - page),
// which is unique per page: the k largest composites are "largest score first, ties
// to the lowest page number".
#include "ktk_common.cuh"
#include "ktk_decode.cuh"
#include "ktk_pipeline.cuh"

namespace ktk {

constexpr int kSelWarps = 8;                        // consumer warps
constexpr int kSelThreads = kSelWarps * 32;         // threads that score and select
constexpr int kSelCtaThreads = kSelThreads + 32;    // + one producer warp
constexpr int kSelStages = 8;                       // one stage per consumer warp
template <typename T> struct SelStage;              // rows per stage: a multiple of the 8 rows a warp scores per step
template <> struct SelStage<__nv_bfloat16> { static constexpr int kRows = 24; };   // 6 KiB
template <> struct SelStage<float> { static constexpr int kRows = 16; };           // 8 KiB
constexpr int kSelCtasPerSm = 3;
constexpr int kMaxTopk = 1024;
constexpr int kSelBins = 2048;                      // first radix digit: the top 11 bits of a key
constexpr int kSelBinShift = 21;
constexpr int kCandMax = 512;                       // pages of the threshold bin ranked directly
static_assert(kSelBins == 8 * kSelThreads, "eight bins per thread in the digit search");
static_assert(kSelStages % kSelWarps == 0, "a stage must belong to one consumer warp");

__device__ __forceinline__ unsigned long long composite(uint32_t key, int page) {
    return ((unsigned long long)key << 16) | (unsigned long long)(0xFFFFu - (unsigned)page);
}

__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kSelThreads) : "memory");
}

// eight consecutive elements (one chunk) of a staged row as fp32
__device__ __forceinline__ void lds8(const float* p, float (&out)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void lds8(const __nv_bfloat16* p, float (&out)[8]) {
    unpack8(*reinterpret_cast<const uint4*>(p), out);
}

// The view of the page table a launch works under (ktk_view with defaults filled in) and the
// width of an output row.
struct SelView {
    int sink_tokens, local_tokens, row_width;
    const int32_t* page_count;
    const int32_t* slot_index;
    const int32_t* seq_order;
};

// What both the producer and the consumers derive for a work item (sequence b, kv head h).
// Scored page r (0 <= r < n_scored) is logical page front + r of the sequence.
struct SelItem {
    int beg, n_pages, front, n_scored, back, n_stages, slot;
    bool bad, need_select, scan;
};

template <int kRowsPerStage>
__device__ __forceinline__ SelItem sel_item(int b, const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                            const SelView& view, int64_t summary_stride, int key_cap, int topk,
                                            bool want_scores) {
    SelItem it;
    const PageSplit ps = page_split(kv_indptr, view.page_count, kv_last_page_len, b, view.sink_tokens,
                                    view.local_tokens);
    it.beg = kv_indptr[b];
    it.slot = view.slot_index ? view.slot_index[b] : b;
    it.n_pages = ps.n_pages;
    it.front = ps.front;
    it.n_scored = ps.n_dyn;
    it.back = ps.back;
    it.bad = ps.bad || (ps.n_pages > 0 && (it.front + it.n_scored > summary_stride || it.n_scored > key_cap ||
                                           it.slot < 0));
    it.need_select = !it.bad && it.n_scored > topk;
    it.scan = it.n_pages > 0 && !it.bad && (it.need_select || want_scores) && it.n_scored > 0;
    it.n_stages = it.scan ? (it.n_scored + kRowsPerStage - 1) / kRowsPerStage : 0;
    return it;
}

// The item CTA `cta` handles in its round `round`, or -1 when that round has none for it.  Without an order: item
// round * grid + cta.  With one (sequences sorted from the longest to the shortest) the rounds alternate in
// direction, so that the CTA that got the longest sequences of one round gets the shortest of the next, and the
// item is (seq_order[rank / Hkv], rank % Hkv); -2 for an entry that is no sequence of the batch.
__device__ __forceinline__ int64_t sel_item_of(int64_t round, int64_t n_items, int Hkv, const int32_t* seq_order) {
    const int64_t grid = gridDim.x, cta = blockIdx.x;
    if (seq_order == nullptr) {
        const int64_t bh = round * grid + cta;
        return bh < n_items ? bh : -1;
    }
    const int64_t rank = round * grid + ((round & 1) ? grid - 1 - cta : cta);
    if (rank >= n_items) return -1;
    const int64_t b = seq_order[rank / Hkv];
    if (b < 0 || b >= n_items / Hkv) return -2;
    return b * Hkv + rank % Hkv;
}

// Persistent kernel: CTA c handles the (sequence, kv head) items c, c + gridDim.x, ... (see sel_item_of)
// A producer warp streams the summaries of its items, one after the other without a gap,
// through a ring of shared-memory stages with bulk asynchronous copies (the rows of one item
// are contiguous); stage i of the stream is scored by consumer warp i mod 8, sixteen lanes per
// row.  While the consumers run the selection of one item, the producer is already filling the
// ring with the rows of the next.  The first radix pass is histogrammed while scoring.
template <typename T, int G>
__global__ void __launch_bounds__(kSelCtaThreads, kSelCtasPerSm)
select_kernel(const T* __restrict__ q, const T* __restrict__ summaries, int64_t summary_stride,
              const int32_t* __restrict__ kv_indices, const int32_t* __restrict__ kv_indptr,
              const int32_t* __restrict__ kv_last_page_len, int topk, int key_cap, int kp, const SelView view,
              int32_t* __restrict__ out_pages, int32_t* __restrict__ out_logical,
              float* __restrict__ out_scores, int64_t n_items, int Hkv, int64_t num_pages,
              int32_t* status) {
    // [stages][6 KiB] | one key per scored page | kp selected composites
    extern __shared__ __align__(128) uint8_t sel_smem[];
    __shared__ __align__(8) uint64_t full_bar[kSelStages];
    __shared__ __align__(8) uint64_t empty_bar[kSelStages];
    __shared__ float qbar[kHeadDim];
    __shared__ unsigned int hist[kSelBins];              // first radix digit, filled while scoring
    __shared__ unsigned long long candc[kCandMax];       // composites of the threshold bin
    __shared__ unsigned int s_wsum[kSelWarps];
    __shared__ int s_digit, s_greater, s_bincount, s_count, s_ccount;
    __shared__ int abort_flag, issued_total;

    constexpr int kRowBytes = kHeadDim * (int)sizeof(T);
    constexpr int kRowsPerStage = SelStage<T>::kRows;
    constexpr int kSelStageBytes = kRowsPerStage * kRowBytes;
    static_assert(kRowsPerStage % 8 == 0, "eight rows per warp step");
    unsigned long long* sel = reinterpret_cast<unsigned long long*>(sel_smem + kSelStages * kSelStageBytes);
    uint32_t* keys = reinterpret_cast<uint32_t*>(sel + kp);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int stride_out = view.row_width;
    const bool want_scores = out_scores != nullptr;

    if (tid == 0) {
        for (int s = 0; s < kSelStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        abort_flag = 0;
        issued_total = 0;
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == kSelWarps) {
        // ---------------- producer warp: one lane issues the bulk copies ----------------
        if (lane == 0) {
            int i = 0;           // stages issued so far, over all items of this CTA
            bool alive = true;
            const int64_t rounds = (n_items + gridDim.x - 1) / gridDim.x;
            for (int64_t round = 0; round < rounds && alive; ++round) {
                const int64_t bh = sel_item_of(round, n_items, Hkv, view.seq_order);
                if (bh < 0) continue;
                const int b = (int)(bh / Hkv);
                const int h = (int)(bh % Hkv);
                const SelItem it = sel_item<kRowsPerStage>(b, kv_indptr, kv_last_page_len, view, summary_stride,
                                                           key_cap, topk, want_scores);
                const T* sbase = summaries + (((int64_t)it.slot * Hkv + h) * summary_stride + it.front) * kHeadDim;
                for (int st = 0; st < it.n_stages; ++st, ++i) {
                    const int s = i % kSelStages;
                    if (i >= kSelStages && !mbar_wait(&empty_bar[s], ((i / kSelStages) - 1) & 1, &abort_flag)) {
                        alive = false;
                        break;
                    }
                    const int r0 = st * kRowsPerStage;
                    const int rows = (it.n_scored - r0 < kRowsPerStage) ? it.n_scored - r0 : kRowsPerStage;
                    const uint32_t bytes = (uint32_t)rows * kRowBytes;
                    mbar_arrive_expect_tx(&full_bar[s], bytes);
                    bulk_load(sel_smem + s * kSelStageBytes, sbase + (int64_t)r0 * kHeadDim, bytes, &full_bar[s]);
                }
            }
            issued_total = i;
        }
    } else {
        // ---------------- consumer warps ----------------
        int ibase = 0;           // stream position of the current item's first stage
        const int64_t rounds = (n_items + gridDim.x - 1) / gridDim.x;
        for (int64_t round = 0; round < rounds; ++round) {
            const int64_t bh = sel_item_of(round, n_items, Hkv, view.seq_order);
            if (bh < 0) {
                if (bh == -2 && tid == 0) report(status, KTK_STATUS_BAD_TABLE);
                continue;
            }
            const int b = (int)(bh / Hkv), h = (int)(bh % Hkv);
            int32_t* row_pages = out_pages + bh * stride_out;
            int32_t* row_logical = out_logical ? out_logical + bh * stride_out : nullptr;
            const SelItem it = sel_item<kRowsPerStage>(b, kv_indptr, kv_last_page_len, view, summary_stride, key_cap,
                                                       topk, want_scores);
            if (it.n_pages <= 0 || it.bad) {
                if (it.bad && tid == 0) report(status, KTK_STATUS_BAD_TABLE);
                for (int i = tid; i < stride_out; i += kSelThreads) {
                    row_pages[i] = -1;
                    if (row_logical) row_logical[i] = -1;
                }
                continue;
            }

            if (it.scan) {
#pragma unroll
                for (int i = 0; i < kSelBins / kSelThreads; ++i) hist[tid + i * kSelThreads] = 0;
                if (tid == 0) { s_count = 0; s_ccount = 0; }
                if (tid < kHeadDim) {
                    const T* qp = q + ((int64_t)b * Hkv * G + (int64_t)h * G) * kHeadDim + tid;
                    float acc = 0.0f;
#pragma unroll
                    for (int g = 0; g < G; ++g) acc = __fadd_rn(acc, to_f32(qp[g * kHeadDim]));
                    qbar[tid] = __fmul_rn(acc, 1.0f / (float)G);
                }
                consumer_sync();
                // Four lanes per row: lane j of a row owns the 8-element chunks j, j+4, j+8, j+12, i.e. the
                // chunks whose partial sums meet in the first two levels of the contract's butterfly, so
                // those two levels are plain in-lane adds and only two shuffles per row remain.  Odd rows
                // visit their chunks rotated by one (bank conflicts); every add involved is commutative,
                // so the value is the same bit for bit.
                const int rw = lane >> 2, j4 = lane & 3, rot = rw & 1;
                const int c0 = (j4 + 4 * ((0 + rot) & 3)) * 8, c1 = (j4 + 4 * ((1 + rot) & 3)) * 8;
                const int c2 = (j4 + 4 * ((2 + rot) & 3)) * 8, c3 = (j4 + 4 * ((3 + rot) & 3)) * 8;
                float q0[8], q1[8], q2[8], q3[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    q0[e] = qbar[c0 + e]; q1[e] = qbar[c1 + e]; q2[e] = qbar[c2 + e]; q3[e] = qbar[c3 + e];
                }
                float* score_row = want_scores ? out_scores + bh * summary_stride + it.front : nullptr;
                // this warp's stages of the item: stream positions i = warp (mod 8) inside [ibase, ibase + n_stages)
                int i = ibase + ((warp - ibase) & (kSelWarps - 1));
                bool ok = true;
                for (; i < ibase + it.n_stages; i += kSelWarps) {
                    const int s = i % kSelStages;
                    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i / kSelStages) & 1, &abort_flag))) {
                        ok = false;
                        break;
                    }
                    const T* stage = reinterpret_cast<const T*>(sel_smem + s * kSelStageBytes);
                    const int r0 = (i - ibase) * kRowsPerStage;
                    constexpr int kSteps = kRowsPerStage / 8;
                    static_assert(kSteps <= 4, "one lane of a row group finishes one step's scores");
                    float accs[kSteps];
#pragma unroll
                    for (int step = 0; step < kSteps; ++step) {
                        const int lr = step * 8 + rw;                 // row inside the stage
                        const T* rowp = stage + lr * kHeadDim;        // rows past the item's last hold stale data: unused
                        float x0[8], x1[8], x2[8], x3[8];
                        lds8(rowp + c0, x0);
                        lds8(rowp + c1, x1);
                        lds8(rowp + c2, x2);
                        lds8(rowp + c3, x3);
                        float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;   // the lane's four chunk chains
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            p0 = __fmaf_rn(q0[e], x0[e], p0);
                            p1 = __fmaf_rn(q1[e], x1[e], p1);
                            p2 = __fmaf_rn(q2[e], x2[e], p2);
                            p3 = __fmaf_rn(q3[e], x3[e], p3);
                        }
                        // butterfly levels "xor 8" (p0 + p2, p1 + p3) and "xor 4", in the lane
                        float acc = __fadd_rn(__fadd_rn(p0, p2), __fadd_rn(p1, p3));
                        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
                        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
                        accs[step] = __fadd_rn(acc, 0.0f);
                    }
                    // all four lanes of a row group hold the same totals: lane j4 finishes step j4
                    // (key, histogram, stores), so that this tail runs once per stage
                    float mine = accs[0];
#pragma unroll
                    for (int step = 1; step < kSteps; ++step) mine = (j4 == step) ? accs[step] : mine;
                    const int r = r0 + j4 * 8 + rw;
                    if (j4 < kSteps && r < it.n_scored) {
                        const uint32_t key = score_to_key(mine);
                        keys[r] = key;
                        if (it.need_select) atomicAdd(&hist[key >> kSelBinShift], 1u);
                        if (score_row) score_row[r] = mine;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_bar[s]);
                }
                ibase += it.n_stages;
                consumer_sync();            // every key of the item is in shared memory (or the CTA gave up)
                if (!ok || abort_flag) break;
            }

            if (!it.need_select) {
                // every scored page is taken, in page order, then the page being filled
                for (int i = tid; i < stride_out; i += kSelThreads) {
                    int logical = -1, phys = -1;
                    if (i < it.n_pages) {
                        logical = i;
                        phys = kv_indices[it.beg + i];
                        if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
                    }
                    row_pages[i] = phys;
                    if (row_logical) row_logical[i] = logical;
                }
                continue;
            }

            // ---- the k-th largest 48-bit composite.  First digit: the top 11 bits of the key (sign,
            //      exponent, two mantissa bits), histogrammed while scoring.  Thread t owns bins
            //      2047-8t .. 2040-8t; a block-wide scan finds the bin in which the k-th largest falls.
            {
                unsigned cnt[8];
                unsigned mine = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    cnt[j] = hist[kSelBins - 1 - 8 * tid - j];
                    mine += cnt[j];
                }
                unsigned incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                if (lane == 31) s_wsum[warp] = incl;
                consumer_sync();
                unsigned running = incl - mine;   // elements in strictly larger bins
                for (int w = 0; w < warp; ++w) running += s_wsum[w];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (running < (unsigned)topk && (unsigned)topk <= running + cnt[j]) {
                        s_digit = kSelBins - 1 - 8 * tid - j;
                        s_greater = (int)running;
                        s_bincount = (int)cnt[j];
                    }
                    running += cnt[j];
                }
                consumer_sync();
            }
            const int digit = s_digit, greater = s_greater, bincount = s_bincount;
            if (bincount <= kCandMax) {
                // ---- usual case: pages with a larger digit are winners; the few pages of the threshold
                //      bin are ranked among themselves and the best (topk - greater) of them join.
                for (int i = tid; i < it.n_scored; i += kSelThreads) {
                    const uint32_t key = keys[i];
                    const int dg = (int)(key >> kSelBinShift);
                    if (dg > digit) {
                        sel[atomicAdd(&s_count, 1)] = composite(key, i);
                    } else if (dg == digit) {
                        candc[atomicAdd(&s_ccount, 1)] = composite(key, i);
                    }
                }
                consumer_sync();
                const int need = topk - greater;
                for (int c = tid; c < bincount; c += kSelThreads) {
                    const unsigned long long mine = candc[c];
                    int rank = 0;
                    for (int j = 0; j < bincount; ++j) rank += (candc[j] > mine) ? 1 : 0;
                    if (rank < need) sel[greater + rank] = mine;
                }
            } else {
                // ---- many pages share the threshold bin (near-equal scores): radix select on the whole
                //      composite, 8 bits per pass ----
                unsigned long long prefix = 0, mask = 0;
                int need = topk;
                for (int shift = 40; shift >= 0; shift -= 8) {
                    hist[tid] = 0;
                    consumer_sync();
                    for (int i = tid; i < it.n_scored; i += kSelThreads) {
                        const unsigned long long c = composite(keys[i], i);
                        if ((c & mask) == prefix) atomicAdd(&hist[(unsigned)(c >> shift) & 255u], 1u);
                    }
                    consumer_sync();
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
                        unsigned running = incl - mine;
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
                    consumer_sync();
                    need -= s_greater;
                    prefix |= (unsigned long long)s_digit << shift;
                    mask |= 0xFFull << shift;
                    if (s_bincount == need) break;   // the whole bin is taken: threshold found
                }
                for (int i = tid; i < it.n_scored; i += kSelThreads) {
                    const unsigned long long c = composite(keys[i], i);
                    if ((c & mask) >= prefix) {
                        const int pos = atomicAdd(&s_count, 1);
                        if (pos < kp) sel[pos] = c;
                    }
                }
            }
            for (int i = topk + tid; i < kp; i += kSelThreads) sel[i] = 0ull;
            consumer_sync();

            // ---- order the winners, best first, and write the row:
            //      [sink page][picks][always-attended tail pages], then -1 ----
            if (topk <= kSelThreads / 2) {
                // the composites are distinct, so the number of larger ones is the position;
                // two threads per winner, half of the comparisons each
                const int e = tid >> 1, hf = tid & 1;
                int rank = 0;
                unsigned long long mine = 0ull;
                if (e < topk) {
                    mine = sel[e];
                    const int j0 = hf ? (topk + 1) / 2 : 0, j1 = hf ? topk : (topk + 1) / 2;
                    for (int j = j0; j < j1; ++j) rank += (sel[j] > mine) ? 1 : 0;
                }
                rank += __shfl_xor_sync(0xffffffffu, rank, 1);
                if (e < topk && hf == 0) {
                    const int logical = it.front + (int)(0xFFFFu - (unsigned)(mine & 0xFFFFull));
                    const int phys = kv_indices[it.beg + logical];
                    if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
                    row_pages[it.front + rank] = phys;
                    if (row_logical) row_logical[it.front + rank] = logical;
                }
            } else {
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
                        consumer_sync();
                    }
                }
                for (int i = tid; i < topk; i += kSelThreads) {
                    const int logical = it.front + (int)(0xFFFFu - (unsigned)(sel[i] & 0xFFFFull));
                    const int phys = kv_indices[it.beg + logical];
                    if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
                    row_pages[it.front + i] = phys;
                    if (row_logical) row_logical[it.front + i] = logical;
                }
            }
            for (int i = tid; i < stride_out; i += kSelThreads) {
                if (i >= it.front && i < it.front + topk) continue;       // the picks, written above
                int logical = -1, phys = -1;
                if (i < it.front) logical = 0;
                else if (i < it.front + topk + it.back) logical = it.front + it.n_scored + (i - it.front - topk);
                if (logical >= 0) {
                    phys = kv_indices[it.beg + logical];
                    if (phys < 0 || phys >= num_pages) report(status, KTK_STATUS_BAD_PAGE);
                }
                row_pages[i] = phys;
                if (row_logical) row_logical[i] = logical;
            }
            consumer_sync();                // sel / keys / hist are reused by the next item
        }
    }

    __syncthreads();
    if (abort_flag && tid == 0) {
        report(status, KTK_STATUS_TIMEOUT);
        volatile int never = 0;   // copies still in flight must land before the shared memory is released
        const int total = issued_total;
        for (int i = (total > kSelStages ? total - kSelStages : 0); i < total; ++i)
            mbar_wait(&full_bar[i % kSelStages], (i / kSelStages) & 1, &never);
    }
}

template <typename T, int G>
static int select_launch(const void* q, const void* summaries, int64_t summary_stride,
                         const int32_t* kv_indices, const int32_t* kv_indptr,
                         const int32_t* kv_last_page_len, int topk, SelView view, int32_t* out_pages,
                         int32_t* out_logical, float* out_scores, const ktk_shape* s,
                         int32_t* status, cudaStream_t st) {
    int key_cap = (int)(summary_stride < kMaxScoredPages ? summary_stride : kMaxScoredPages);
    int kp = 1;
    while (kp < topk) kp <<= 1;
    const size_t smem = (size_t)kSelStages * SelStage<T>::kRows * kHeadDim * sizeof(T) + (size_t)kp * 8 +
                        (size_t)key_cap * sizeof(uint32_t);
    auto kern = select_kernel<T, G>;
    KTK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                 "ktk_select");
    const int64_t items = (int64_t)s->batch * s->num_kv_heads;
    int64_t grid = (int64_t)sm_count() * kSelCtasPerSm;
    if (grid > items) grid = items;
    kern<<<(unsigned)grid, kSelCtaThreads, smem, st>>>(
        (const T*)q, (const T*)summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
        topk, key_cap, kp, view, out_pages, out_logical, out_scores, items, s->num_kv_heads, s->num_pages,
        status);
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

extern "C" int ktk_select_v(const void* q, const void* summaries, int64_t summary_stride,
                            const int32_t* kv_indices, const int32_t* kv_indptr,
                            const int32_t* kv_last_page_len, int32_t topk, const ktk_view* view_in,
                            int32_t row_width, int32_t* out_pages, int32_t* out_logical, float* out_scores,
                            const ktk_shape* shape, int32_t* status, void* stream) {
    int rc = check_shape(shape, "ktk_select");
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, "ktk_select");
    if (rc != KTK_OK) return rc;
    if (topk < 1 || topk > kMaxTopk) {
        set_error("ktk_select: topk %d outside [1, %d]", topk, kMaxTopk);
        return topk < 1 ? KTK_ERR_ARG : KTK_ERR_TOO_LARGE;
    }
    const View v = make_view(view_in);
    const int need_width = view_row_width(topk, v);
    if (row_width == 0) row_width = need_width;
    if (row_width < need_width) {
        set_error("ktk_select: output rows of %d entries, this view needs %d", row_width, need_width);
        return KTK_ERR_ARG;
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
    if (((uintptr_t)summaries & 15u) != 0) {
        set_error("ktk_select: summaries must be 16-byte aligned (bulk asynchronous copies)");
        return KTK_ERR_ARG;
    }
    if ((int64_t)shape->batch * shape->num_kv_heads > 2147483647LL) {
        set_error("ktk_select: batch * num_kv_heads exceeds the grid limit");
        return KTK_ERR_TOO_LARGE;
    }
    SelView sv;
    sv.sink_tokens = v.sink_tokens; sv.local_tokens = v.local_tokens; sv.row_width = row_width;
    sv.page_count = v.page_count; sv.slot_index = v.slot_index; sv.seq_order = v.seq_order;
    cudaStream_t st = (cudaStream_t)stream;
    if (shape->dtype == KTK_F32)
        return select_group<float>(shape->group_size, q, summaries, summary_stride, kv_indices,
                                   kv_indptr, kv_last_page_len, (int)topk, sv, out_pages, out_logical,
                                   out_scores, shape, status, st);
    return select_group<__nv_bfloat16>(shape->group_size, q, summaries, summary_stride, kv_indices,
                                       kv_indptr, kv_last_page_len, (int)topk, sv, out_pages,
                                       out_logical, out_scores, shape, status, st);
}

extern "C" int ktk_select(const void* q, const void* summaries, int64_t summary_stride,
                          const int32_t* kv_indices, const int32_t* kv_indptr,
                          const int32_t* kv_last_page_len, int32_t topk, int32_t* out_pages,
                          int32_t* out_logical, float* out_scores, const ktk_shape* shape,
                          int32_t* status, void* stream) {
    return ktk_select_v(q, summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len, topk, nullptr, 0,
                        out_pages, out_logical, out_scores, shape, status, stream);
}
