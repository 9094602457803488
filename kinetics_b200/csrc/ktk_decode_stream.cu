// Paged flash-decode attention, bf16 tensor cores, balanced partition of the page lists.
//
// The per-unit kernel (ktk_decode_mma.cu) launches one CTA per (sequence, kv head): with
// 4096 units on 444 resident CTAs the last wave runs 22 % full, and every CTA pays the fill
// and the drain of its pipeline.  Here the grid is one CTA per resident slot and the
// concatenation of all page lists is cut into equal chunks instead:
//
//   position = unit * wmax + entry        unit = b * Hkv + h,  wmax = entries per list (padded)
//   CTA c owns positions [c * chunk, (c + 1) * chunk)
//
// (dense CSR lists are cut entry by entry instead, position = (indptr[b] - indptr[0]) * Hkv + h * n(b)
// + entry, so that batches of very different lengths are balanced as well)
//
// so a CTA runs a few whole units and at most two pieces of units that cross into a neighbour.
// The producer warp keeps the TMA ring full across unit boundaries; the four consumer warps
// merge at the end of each unit (through 8 KiB of shared memory next to the ring) and write
// either the output row (the CTA saw every entry of the unit) or an un-normalised partial
// (m, l, O) into one of the CTA's two workspace slots: "tail" for a unit that starts in this
// CTA and continues into the next, "head" for a unit that started in an earlier CTA.
// stream_combine_kernel then merges the pieces of every cut unit (at most one per CTA).
// Which CTA holds which piece follows from the shapes alone, so results are deterministic.
#include <cstdlib>
#include <mutex>

#include "ktk_decode_mma.cuh"

namespace ktk {

constexpr int kStreamMaxCtasPerSm = 4;                    // the most any variant keeps resident (sizes the workspace)
constexpr int kStreamMinChunk = 16;                       // pages: below this a CTA is not worth its start-up
constexpr int kExchangeHeads = 4;                         // heads merged per pass through shared memory
constexpr int kExchangeBytes = kMmaConsumers * kExchangeHeads * kHeadDim * 4;   // 8 KiB
constexpr int stream_smem(int stages) { return stages * kStageBytes + 1024 + kExchangeBytes; }

struct StreamParams {
    DecodeParams d;
    int G;
    int wmax;        // padded mode: positions per unit
    int chunk;       // padded mode: positions per CTA
    int64_t total;   // padded mode: units * wmax
    int exact;       // 1: dense CSR lists without a page_count view -- positions are the CSR entries themselves,
                     //    unit (b, h) covers [(indptr[b] - indptr[0]) * Hkv + h * n(b), ... + n(b)), so ragged
                     //    batches are cut evenly too; total and chunk are computed on the device
};

// positions [p0, p1) of CTA c; empty if p1 <= p0
struct Range {
    int64_t p0, p1;
};

// number of positions and positions per CTA
__device__ __forceinline__ void stream_extent(const StreamParams& p, int64_t& total, int64_t& chunk) {
    total = p.total;
    chunk = p.chunk;
    if (p.exact) {
        total = (int64_t)(p.d.kv_indptr[p.d.batch] - p.d.kv_indptr[0]) * p.d.Hkv;
        chunk = (total + gridDim.x - 1) / gridDim.x;
        if (chunk < kStreamMinChunk) chunk = kStreamMinChunk;
    }
}

__device__ __forceinline__ Range cta_range(const StreamParams& p, int64_t c) {
    Range r;
    int64_t total, chunk;
    stream_extent(p, total, chunk);
    r.p0 = c * chunk;
    r.p1 = (r.p0 + chunk < total) ? r.p0 + chunk : total;
    return r;
}

// The unit (b, h) whose positions are [start, start + len)
struct Cursor {
    int b, h, len;
    int64_t start;
};

// exact mode: the sequence whose CSR entries contain entry q (relative to indptr[0]); all lanes of the
// warp take part, 32 probes per round
__device__ __forceinline__ int find_sequence(const int32_t* indptr, int B, int64_t q) {
    const int lane = threadIdx.x & 31;
    const int64_t base = indptr[0];
    int lo = 0, hi = B;                                   // invariant: indptr[lo] - base <= q, answer in [lo, hi)
    while (hi - lo > 1) {
        const int step = (hi - lo + 31) / 32;
        const int idx = lo + lane * step;
        const bool ok = idx < hi && (int64_t)indptr[idx] - base <= q;
        const unsigned m = __ballot_sync(0xffffffffu, ok);            // a prefix of the lanes: lane 0 always holds
        const int k = 31 - __clz((int)m);
        lo += k * step;
        hi = (lo + step < hi) ? lo + step : hi;
    }
    return lo;
}

__device__ __forceinline__ Cursor cursor_at(const StreamParams& p, int64_t pos) {
    Cursor c;
    if (!p.exact) {
        const int64_t u = pos / p.wmax;
        c.b = (int)(u / p.d.Hkv);
        c.h = (int)(u % p.d.Hkv);
        c.start = u * p.wmax;
        c.len = p.wmax;
        return c;
    }
    const int32_t* ip = p.d.kv_indptr;
    c.b = find_sequence(ip, p.d.batch, pos / p.d.Hkv);
    c.len = ip[c.b + 1] - ip[c.b];
    const int64_t first = (int64_t)(ip[c.b] - ip[0]) * p.d.Hkv;
    c.h = (int)((pos - first) / c.len);
    c.start = first + (int64_t)c.h * c.len;
    return c;
}

__device__ __forceinline__ void cursor_next(const StreamParams& p, Cursor& c) {
    c.start += c.len;
    if (++c.h < p.d.Hkv) return;
    c.h = 0;
    ++c.b;
    if (p.exact) {
        while (c.b < p.d.batch && (c.len = p.d.kv_indptr[c.b + 1] - p.d.kv_indptr[c.b]) == 0) ++c.b;   // no positions
    }
}

// The part of the cursor's unit that falls into the position range [p0, p1).
struct Piece {
    int b, h;
    EntryList el;
    int e_lo, e_hi;   // entries of the unit this CTA runs
    bool first;       // the unit's positions start inside the range
    bool bad;
};

__device__ __forceinline__ Piece get_piece(const StreamParams& p, const Cursor& c, int64_t p0, int64_t p1) {
    Piece pc;
    pc.b = c.b;
    pc.h = c.h;
    pc.el = entry_list(p.d, pc.b, pc.h, pc.bad);
    if (pc.el.cnt > c.len) {          // a list longer than the caller's bound: flagged by the producer, clipped here
        pc.el.cnt = c.len;
        pc.bad = true;
    }
    const int lo = (p0 > c.start) ? (int)(p0 - c.start) : 0;
    const int hi = (p1 - c.start < c.len) ? (int)(p1 - c.start) : c.len;
    pc.first = (p0 <= c.start);
    pc.e_lo = lo < pc.el.cnt ? lo : pc.el.cnt;
    pc.e_hi = hi < pc.el.cnt ? hi : pc.el.cnt;
    return pc;
}

__device__ __forceinline__ void consumer_bar() {          // the four consumer warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kMmaConsumers * 32) : "memory");
}

// STAGES: ring depth (a multiple of the consumer count, so that a stage always belongs to one warp);
// CTAS: CTAs resident per SM.
template <int STAGES, int CTAS>
__global__ void __launch_bounds__(kMmaThreads, CTAS)
decode_stream_kernel(const StreamParams p, const __grid_constant__ CUtensorMap kv_map) {
    static_assert(STAGES % kMmaConsumers == 0, "a stage must belong to one consumer warp");
    constexpr int kMmaStages = STAGES;                     // shadows the per-list kernel's ring depth
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMmaStages];
    __shared__ __align__(8) uint64_t empty_bar[kMmaStages];
    __shared__ int stage_tag[kMmaStages];     // issue index + 1 of the page in the stage, negated if skipped
    __shared__ int abort_flag;
    __shared__ int issued_total;
    __shared__ float red_m[kMmaConsumers][8], red_l[kMmaConsumers][8];

    // the swizzle pattern is a function of the shared-memory address: stages start on 1 KiB
    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* red_o = reinterpret_cast<float*>(stages + kMmaStages * kStageBytes);   // [warp][head of the pass][128]

    const DecodeParams& d = p.d;
    const int G = p.G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hq = d.Hkv * G;
    const Range rg = cta_range(p, blockIdx.x);
    if (rg.p1 <= rg.p0) return;                            // nothing left for this CTA (exact mode, small batches)
    const int64_t p0 = rg.p0, p1 = rg.p1;

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

    if (warp == kMmaConsumers) {
        // ---------------- producer warp: one ring across all of the CTA's units ----------------
        if (lane == 0) prefetch_tensormap(&kv_map);
        int issued = 0;
        bool alive = true;
        for (Cursor cur = cursor_at(p, p0); cur.start < p1 && cur.b < d.batch && alive; cursor_next(p, cur)) {
            const Piece pc = get_piece(p, cur, p0, p1);
            if (pc.bad && pc.first && lane == 0) report(d.status, KTK_STATUS_BAD_TABLE);
            const int e0 = pc.e_lo, e1 = pc.e_hi;
            int next_ids = (e0 + lane < e1) ? pc.el.ptr[e0 + lane] : -1;
            for (int base = e0; base < e1 && alive; base += 32) {
                const int ids = next_ids;
                next_ids = (base + 32 + lane < e1) ? pc.el.ptr[base + 32 + lane] : -1;   // one chunk ahead
                const int n = (e1 - base < 32) ? e1 - base : 32;
                for (int j = 0; j < n && alive; ++j) {
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
                            tma_load_page(stages + s * kStageBytes, &kv_map, &full_bar[s], page, pc.h);
                            issued = i + 1;
                        }
                    }
                    alive = __shfl_sync(0xffffffffu, (int)alive, 0) != 0;
                }
            }
        }
        if (lane == 0) issued_total = issued;
    } else {
        // ---------------- consumer warps ----------------
        const int gid = lane >> 2, tig = lane & 3;
        MmaState ms;
        int base_i = 0;            // issue index of the unit's first page
        bool dead = false;         // gave up: keep walking (the barriers below must stay matched), compute nothing
        for (Cursor cur = cursor_at(p, p0); cur.start < p1 && cur.b < d.batch; cursor_next(p, cur)) {
            const Piece pc = get_piece(p, cur, p0, p1);
            const int n = pc.e_hi - pc.e_lo;
            // what this CTA owes the unit: nothing, the output row, or a partial in its tail / head slot
            const bool whole = pc.first && pc.e_hi == pc.el.cnt;
            const bool partial = !whole && (pc.first || n > 0);
            if (!whole && !partial) continue;
            ms.reset();
            if (n > 0 && !dead) {
                uint32_t qb[8][2];
                load_q_frags(qb, d.q, (int64_t)pc.b * Hq + (int64_t)pc.h * G, G, lane);
                for (int j = (warp - base_i) & (kMmaConsumers - 1); j < n; j += kMmaConsumers) {
                    const int i = base_i + j;
                    const int s = i % kMmaStages;
                    // the vote keeps the warp together should a single lane give up
                    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], (i / kMmaStages) & 1, &abort_flag))) {
                        dead = true;
                        break;
                    }
                    const int tag = stage_tag[s];
                    if (tag != i + 1 && tag != -(i + 1)) {
                        // the stage does not hold the page this warp is waiting for: stop rather than compute on it
                        if (lane == 0) { report(d.status, KTK_STATUS_INTERNAL); abort_flag = 1; }
                        dead = true;
                        break;
                    }
                    if (tag > 0)
                        mma_consume_page(ms, stages + s * kStageBytes, entry_tokens(pc.el, pc.e_lo + j), qb,
                                         d.scale_log2, lane);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_bar[s]);
                }
            }
            base_i += n;

            // ---- end of the unit: merge the four warps, kExchangeHeads heads per pass ----
            if (gid == 0) {
                red_m[warp][2 * tig] = ms.m0; red_m[warp][2 * tig + 1] = ms.m1;
                red_l[warp][2 * tig] = ms.l0; red_l[warp][2 * tig + 1] = ms.l1;
            }
            const int slot = blockIdx.x * 2 + (pc.first ? 1 : 0);      // head slot 0, tail slot 1
            for (int pass = 0; pass * kExchangeHeads < G; ++pass) {
                if ((tig >> 1) == pass) {
                    const int hl = 2 * (tig & 1);
#pragma unroll
                    for (int mt = 0; mt < 8; ++mt) {
                        float* o0 = red_o + ((warp * kExchangeHeads + hl) * kHeadDim) + 16 * mt + gid;
                        o0[0] = ms.acc[mt][0];
                        o0[kHeadDim] = ms.acc[mt][1];
                        o0[8] = ms.acc[mt][2];
                        o0[kHeadDim + 8] = ms.acc[mt][3];
                    }
                }
                consumer_bar();
                const int dd = tid;                                    // 128 consumer threads = 128 head dims
                const int g_end = (G < (pass + 1) * kExchangeHeads) ? G : (pass + 1) * kExchangeHeads;
                for (int g = pass * kExchangeHeads; g < g_end; ++g) {
                    float M = red_m[0][g];
#pragma unroll
                    for (int w = 1; w < kMmaConsumers; ++w) M = fmaxf(M, red_m[w][g]);
                    float L = 0.0f, O = 0.0f;
                    if (M != -INFINITY) {
#pragma unroll
                        for (int w = 0; w < kMmaConsumers; ++w) {
                            const float wt = exp2f(red_m[w][g] - M);
                            L += wt * red_l[w][g];
                            O += wt * red_o[(w * kExchangeHeads + (g - pass * kExchangeHeads)) * kHeadDim + dd];
                        }
                    }
                    if (abort_flag) continue;                          // the CTA gave up: write nothing
                    if (whole) {
                        const int64_t qh = (int64_t)pc.b * Hq + (int64_t)pc.h * G + g;
                        ((__nv_bfloat16*)d.o)[qh * kHeadDim + dd] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
                    } else {
                        const int64_t row = (int64_t)slot * G + g;
                        d.ws_o[row * kHeadDim + dd] = O;
                        if (dd == 0) { d.ws_ml[row * 2] = M; d.ws_ml[row * 2 + 1] = L; }
                    }
                }
                consumer_bar();                                        // red_o / red_m are free again
            }
        }
    }

    __syncthreads();   // every page consumed (or the CTA gave up): stage memory is free
    if (abort_flag && tid == 0) {
        report(d.status, KTK_STATUS_TIMEOUT);
        // wait, again bounded, for copies still in flight before the CTA's shared memory is released
        volatile int never = 0;
        const int total = issued_total;
        for (int i = (total > kMmaStages ? total - kMmaStages : 0); i < total; ++i)
            mbar_wait(&full_bar[i % kMmaStages], (i / kMmaStages) & 1, &never);
    }
}

// One CTA per CTA of the decode grid: merges the pieces of the unit that starts in that CTA's
// range and continues beyond it (if there is one), and writes its output rows.  In exact mode it
// also writes the zero rows of sequences without pages (they own no position, so no decode CTA
// meets them).
__global__ void __launch_bounds__(kHeadDim)
stream_combine_kernel(const StreamParams p) {
    const DecodeParams& d = p.d;
    const int G = p.G, dd = threadIdx.x;
    if (p.exact) {
        for (int b = blockIdx.x; b < d.batch; b += gridDim.x) {
            if (d.kv_indptr[b + 1] - d.kv_indptr[b] > 0) continue;
            for (int hq = 0; hq < d.Hkv * G; ++hq)
                ((__nv_bfloat16*)d.o)[((int64_t)b * d.Hkv * G + hq) * kHeadDim + dd] = __float2bfloat16_rn(0.0f);
        }
    }
    const int64_t c = blockIdx.x;
    const Range rg = cta_range(p, c);
    if (rg.p1 <= rg.p0) return;
    int64_t total, chunk;
    stream_extent(p, total, chunk);
    if (rg.p1 >= total) return;                                // the last CTA: nothing continues
    const Cursor cur = cursor_at(p, rg.p1 - 1);                // the last unit of CTA c
    if (cur.start < rg.p0) return;                             // it began in an earlier CTA: merged there
    const Piece pc = get_piece(p, cur, rg.p0, rg.p1);
    if (cur.start + pc.el.cnt <= rg.p1) return;                // every entry of the unit lies in CTA c
    const int64_t end = cur.start + pc.el.cnt;
    for (int g = 0; g < G; ++g) {
        float M = -INFINITY, L = 0.0f, O = 0.0f;
        for (int64_t c2 = c; c2 * chunk < end; ++c2) {
            const int64_t row = (c2 * 2 + (c2 == c ? 1 : 0)) * G + g;   // tail slot of c, head slots after it
            const float m = d.ws_ml[row * 2], l = d.ws_ml[row * 2 + 1];
            if (m == -INFINITY) continue;
            const float Mn = fmaxf(M, m);
            const float a = exp2f(M - Mn), bsc = exp2f(m - Mn);
            L = L * a + l * bsc;
            O = O * a + d.ws_o[row * kHeadDim + dd] * bsc;
            M = Mn;
        }
        const int64_t qh = ((int64_t)pc.b * d.Hkv + pc.h) * G + g;
        ((__nv_bfloat16*)d.o)[qh * kHeadDim + dd] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    }
}

// Ring depth x residency variants.  Which one runs: the environment variable KTK_STREAM_VARIANT (a tuning knob,
// read once), else the measured best for the kind of list.
struct StreamVariant {
    int stages, ctas;
    void (*kernel)(const StreamParams, const CUtensorMap);
};
// Measured on a B200 at B = 4096, 32768-token context (sparse: 129 pages per list / dense: 2049), ms:
//   4 stages x 4 CTAs per SM   0.639 / 9.53      <- default: 16 consumer warps per SM
//   8 stages x 3 CTAs per SM   0.643 / 10.29
//   4 stages x 3 CTAs per SM   0.668 / 10.16
//   4 stages x 5 CTAs per SM   0.714 / 10.96     (72 registers: spills)
//   8 or 12 stages x 2 CTAs    0.88  / 13.5
// The consumer warps, not the bytes in flight, set the pace: more resident warps win until registers run out.
static const StreamVariant kStreamVariants[] = {
    {4, 4, decode_stream_kernel<4, 4>},      // 0
    {8, 3, decode_stream_kernel<8, 3>},      // 1
};
constexpr int kNumStreamVariants = (int)(sizeof(kStreamVariants) / sizeof(kStreamVariants[0]));

static int stream_variant_index(bool dense) {
    static const int forced = [] {
        const char* e = getenv("KTK_STREAM_VARIANT");
        const int v = e ? atoi(e) : -1;
        return (v >= 0 && v < kNumStreamVariants) ? v : -1;
    }();
    if (forced >= 0) return forced;
    (void)dense;
    return 0;
}

// resident CTAs of a variant on the current device
static int stream_slots(int vi) {
    static std::mutex mu;
    static int slots[64][kNumStreamVariants] = {};
    const StreamVariant& v = kStreamVariants[vi];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return v.ctas * sm_count();
    std::lock_guard<std::mutex> lock(mu);
    if (slots[dev][vi] == 0) {
        int per_sm = 0;
        const int smem = stream_smem(v.stages);
        cudaFuncSetAttribute(v.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, v.kernel, kMmaThreads, smem) != cudaSuccess ||
            per_sm < 1)
            per_sm = 1;
        if (per_sm > v.ctas) per_sm = v.ctas;
        slots[dev][vi] = per_sm * sm_count();
    }
    return slots[dev][vi];
}

static int stream_grid_of(int vi, int64_t units, int max_entries) {
    const int64_t total = units * (int64_t)max_entries;
    int64_t grid = (total + kStreamMinChunk - 1) / kStreamMinChunk;
    const int64_t slots = stream_slots(vi);
    if (grid > slots) grid = slots;
    if (grid < 1) grid = 1;
    return (int)grid;
}

int stream_grid(int64_t units, int max_entries) { return stream_grid_of(stream_variant_index(false), units, max_entries); }

size_t stream_workspace_bytes(int G) {
    // two slots per CTA of the largest grid, each G rows of (m, l) + 128 floats
    return (size_t)kStreamMaxCtasPerSm * sm_count() * 2 * G * (2 + kHeadDim) * sizeof(float);
}

int launch_decode_stream(const DecodeParams& p, int G, int max_entries, cudaStream_t st) {
    CUtensorMap map;
    int rc = make_kv_tensor_map(&map, p);
    if (rc != KTK_OK) return rc;
    StreamParams sp;
    sp.d = p;
    sp.G = G;
    sp.wmax = max_entries;
    // dense CSR lists: cut the entries themselves (ragged batches stay balanced); selected-page tables
    // and page_count views: cut the padded rows
    sp.exact = (p.topk < 0 && p.page_count == nullptr) ? 1 : 0;
    const int64_t units = (int64_t)p.batch * p.Hkv;
    sp.total = units * max_entries;
    const int vi = stream_variant_index(p.topk < 0);
    const StreamVariant& var = kStreamVariants[vi];
    int grid = stream_grid_of(vi, units, max_entries);
    const int64_t chunk = (sp.total + grid - 1) / grid;
    if (chunk > 2147483647LL) {
        set_error("ktk decode: %lld page positions per CTA exceed the balanced partition's limit", (long long)chunk);
        return KTK_ERR_TOO_LARGE;
    }
    sp.chunk = (int)chunk;
    if (!sp.exact) grid = (int)((sp.total + chunk - 1) / chunk);            // no empty CTA
    const int smem = stream_smem(var.stages);
    KTK_CUDA_TRY(cudaFuncSetAttribute(var.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "ktk decode (balanced)");
    var.kernel<<<grid, kMmaThreads, smem, st>>>(sp, map);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk decode (balanced)");
    if (grid > 1 || sp.exact) {
        stream_combine_kernel<<<grid, kHeadDim, 0, st>>>(sp);
        KTK_CUDA_TRY(cudaGetLastError(), "ktk decode (balanced, combine)");
    }
    return KTK_OK;
}

}  // namespace ktk
