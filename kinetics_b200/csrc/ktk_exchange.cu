// The two exchanges of the tensor-parallel layer over NVLink, row-pipelined:
//   * o_proj:    all-reduce of the ranks' partial outputs + residual add + RMSNorm
//                (LiteSys/litesys/models/qwen3_dist.py:111-114)
//   * down_proj: all-reduce (or reduce-scatter) of the partial outputs + residual add (:120-122)
//
// Rank r owns the rows [r * rows / world, (r + 1) * rows / world).  CTA c of G walks the owned rows
// c, c + G, ... one after the other:
//     loads of row j+1 are issued (switch-reduced multimem.ld_reduce, or plain peer loads)
//     row j: fp32 sum of the partials + residual, rounded to bf16, sent to every rank
//            (multimem.st or peer stores), normalised from registers into this rank's `norm`
//     fence + flag: "row j of this CTA is on its way", to the same-index CTA of every rank
//     rows that the same-index CTAs of the other ranks have flagged meanwhile are normalised locally
// so that a rank's outbound link (the partials it serves to the others' reductions) and its inbound
// link (the sums the others send) can be busy at the same time, and the local normalisation of the
// received rows hides behind the link time.  In the lock-step form of ktk_comm.cu all CTAs load,
// then all CTAs store, then all normalise.
// Measured on two B200s over 32 MiB (CUDA events, 50 launches): reduce-scatter + residual 46 us (NCCL
// reduce_scatter alone 55 us); all-reduce + residual + norm 109 us here against 79 us for the lock-step
// kernel, whose single fence per CTA costs less than one system-scope release per row -- the lock-step
// kernel therefore stays the default for that result, this kernel serves the other two.
//
// Flags: one word per (CTA, source rank) in every rank's memory, written with st.release.sys by the
// source and polled with ld.acquire.sys; the values only grow (a per-CTA launch counter kept in
// local memory times `stride`), so nothing is reset between launches and the kernel can sit in a
// CUDA graph.  Every poll is bounded; on expiry the CTA records KTK_STATUS_TIMEOUT and goes on.
// No TMA and no bulk copy touches peer memory.
#include "ktk_comm.cuh"

namespace ktk {

constexpr int kXThreads = 512;
constexpr int kXMaxVec = 2;             // vectors of 8 elements per thread: cols <= 8192

__device__ __forceinline__ uint4 ld_cg_16(const void* p) {
    uint4 r;
    // volatile: the loads of the next row must be issued where they are written, ahead of this
    // row's arithmetic and stores
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <int NV, int PEERS>
struct RowLoads {
    uint4 x[NV][PEERS > 0 ? PEERS : 1];
    uint4 t[NV];
};

template <int NV, int PEERS>
__device__ __forceinline__ void issue_row(RowLoads<NV, PEERS>& L, const __nv_bfloat16* x_mc,
                                          const __nv_bfloat16* const* x_peer, const __nv_bfloat16* residual,
                                          int row, int cols, int nvec) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * kXThreads;
        if (c < nvec) {
            const size_t off = (size_t)row * cols + (size_t)c * 8;
            if constexpr (PEERS > 0) {
#pragma unroll
                for (int p = 0; p < PEERS; ++p) L.x[i][p] = ld_cg_16(x_peer[p] + off);
            } else {
                L.x[i][0] = multimem_ld_reduce_bf16x8(x_mc + off);
            }
            L.t[i] = __ldg(reinterpret_cast<const uint4*>(residual + off));
        }
    }
}

template <int NV>
__device__ __forceinline__ void store_norm(const float (&v)[NV][8], float inv, const __nv_bfloat16* __restrict__ w,
                                           __nv_bfloat16* norm_row, int nvec) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * kXThreads;
        if (c < nvec) {
            float wv[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(w + (size_t)c * 8)), wv);
            uint4 packed;
            uint32_t* pw = &packed.x;
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(v[i][e] * inv * wv[e], v[i][e + 1] * inv * wv[e + 1]);
                pw[e / 2] = *reinterpret_cast<const uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(norm_row + (size_t)c * 8) = packed;
        }
    }
}

// ---- CTA-internal hand-off between the data warps and the signalling warp ----
__device__ __forceinline__ void bar_sync_named(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_release_cta_shared(int* p, int v) {
    asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta_shared(const int* p) {
    int v;
    asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_cta_shared_add(int* p, int v) {
    asm volatile("red.release.cta.shared.add.s32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}

constexpr int kXDataWarps = kXThreads / 32;
constexpr int kXAllThreads = kXThreads + 32;     // + the signalling warp

// rows of loads in flight per thread (the ring), by how much of a row a thread holds
template <int NV, int PEERS>
struct XDepth {
    static constexpr int value = (PEERS == 4) ? (NV == 2 ? 2 : 3) : (PEERS == 2 ? (NV == 2 ? 2 : 5) : 3);
    static constexpr int ctas_per_sm = (PEERS == 0 && NV == 1) ? 2 : 1;
};

// NV: vectors per thread.  PEERS = 0: the switch reduces and multicasts; PEERS = world (2 or 4): peer
// loads and stores.  SCATTER: the sums of the owned rows stay on this rank (reduce-scatter), nothing
// is sent and nothing is normalised.  NORM (all-reduce form only): RMSNorm of every row into `norm`.
//
// 16 data warps move rows; a 17th warp does all cross-rank signalling, so that no data warp ever sits in a
// system-scope fence: a data warp that has stored its part of row j adds one to a shared counter (release,
// CTA scope); the signalling warp sees the counter reach 16 * (j + 1) (acquire), then tells every rank "row
// j of this CTA is on its way" (st.release.sys, cumulative over the data warps' stores) and publishes, in
// shared memory, how many rows the same-index CTAs of the other ranks have flagged.
template <int NV, int PEERS, bool SCATTER, bool NORM>
__global__ void __launch_bounds__(kXAllThreads, XDepth<NV, PEERS>::ctas_per_sm)
exchange_rows_kernel(const __nv_bfloat16* x_mc, const __nv_bfloat16* const* x_peer,
                     const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* sum_mc, __nv_bfloat16* const* sum_peer, __nv_bfloat16* sum_local,
                     __nv_bfloat16* norm_local, uint32_t* const* flags, uint32_t* launch_count, int rank, int world,
                     int rows, int cols, float eps, uint32_t stride, int32_t* status) {
    constexpr int DEPTH = XDepth<NV, PEERS>::value;
    __shared__ float part[kXDataWarps];
    __shared__ uint32_t s_epoch;
    __shared__ int s_avail[kCommMaxWorld];      // rows the same-index CTA of rank p has flagged (signalling warp writes)
    __shared__ int s_take[kCommMaxWorld];       // snapshot of s_avail the data warps agree on
    __shared__ int s_done[kCommMaxWorld];       // rows of rank p this CTA has normalised
    __shared__ int s_warps_done;                // data-warp arrivals: 16 per finished row (per kernel for SCATTER)
    if (threadIdx.x == 0) { s_epoch = launch_count[blockIdx.x]; s_warps_done = 0; }
    if (threadIdx.x < kCommMaxWorld) { s_avail[threadIdx.x] = 0; s_take[threadIdx.x] = 0; s_done[threadIdx.x] = 0; }
    __syncthreads();
    const uint32_t base = s_epoch * stride;
    const int G = gridDim.x;
    const int per = rows / world;
    const int nvec = cols / 8;
    const int J = (per - (int)blockIdx.x + G - 1) / G;      // rows of every owner that fall to CTAs of this index
    uint32_t* my_flags = flags[rank] + (size_t)blockIdx.x * world;
    const int lane = threadIdx.x & 31;
    const bool signaller = threadIdx.x >= kXThreads;

    // every rank's partial output is complete (its GEMM precedes this kernel in stream order)
    if (signaller && lane < world) {
        st_release_sys(flags[lane] + (size_t)blockIdx.x * world + rank, base + 1);
        flag_wait(my_flags + lane, base + 1, status);
    }
    __syncthreads();

    if (signaller) {
        // ---------------- the signalling warp ----------------
        int sent = 0;                   // own rows flagged so far (SCATTER: 0 or 1 for the closing flag)
        const int to_send = SCATTER ? 1 : J;
        const int per_flag = SCATTER ? kXDataWarps * 1 : kXDataWarps;
        bool gave_up = false;
        for (uint32_t spin = 0;; ++spin) {
            const int arrived = ld_acquire_cta_shared(&s_warps_done);
            const int ready = SCATTER ? (arrived >= per_flag ? 1 : 0) : arrived / per_flag;
            while (sent < ready) {
                // SCATTER: nobody may overwrite its partial output while a peer still reads it -- one closing flag
                if (lane < world)
                    st_release_sys(flags[lane] + (size_t)blockIdx.x * world + rank, base + 2 + (SCATTER ? 0 : sent));
                ++sent;
            }
            bool in = true;
            if (lane < world) {
                const int32_t got = (int32_t)(ld_acquire_sys(my_flags + lane) - (base + 1));
                const int want = SCATTER ? 1 : J;
                const int have = got < 0 ? 0 : (got > want ? want : got);
                if (!SCATTER) st_release_cta_shared(&s_avail[lane], gave_up ? J : have);
                in = have >= want;
            }
            const bool all_in = __all_sync(0xffffffffu, in) || gave_up;
            if (sent == to_send && all_in) break;
            if (spin > (kCommSpinCap >> 2) && !gave_up) {
                // a peer never arrived: record it, let the data warps run on (they wait for s_avail only)
                if (lane == 0) report(status, KTK_STATUS_TIMEOUT);
                gave_up = true;
            }
            if (spin > 16) __nanosleep(spin > 4096 ? 256 : 32);
        }
        if (lane == 0) launch_count[blockIdx.x] = s_epoch + 1;
        return;
    }

    // ---------------- the data warps ----------------
    auto data_sync = [&]() { bar_sync_named(1, kXThreads); };
    auto inv_rms = [&](float ss) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        data_sync();                                   // `part` of the previous row has been read
        if (lane == 0) part[threadIdx.x >> 5] = ss;
        data_sync();
        float tot = 0.0f;
#pragma unroll
        for (int i = 0; i < kXDataWarps; ++i) tot += part[i];
        return rsqrtf(tot / (float)cols + eps);
    };
    auto norm_received = [&](size_t r) {
        const __nv_bfloat16* sum_row = sum_local + r * cols;
        float v[NV][8];
        float ss = 0.0f;
        uint4 sr[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * kXThreads;
            if (c < nvec) sr[i] = __ldcg(reinterpret_cast<const uint4*>(sum_row + (size_t)c * 8));
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * kXThreads;
            if (c < nvec) {
                unpack8(sr[i], v[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
            }
        }
        const float inv = inv_rms(ss);
        store_norm<NV>(v, inv, w, norm_local + r * cols, nvec);
    };
    // rows another rank has flagged so far: normalise those not yet done (never blocks)
    auto drain = [&]() {
        if ((int)threadIdx.x < world) s_take[threadIdx.x] = ld_acquire_cta_shared(&s_avail[threadIdx.x]);
        data_sync();
        for (int p = 1; p < world; ++p) {
            const int owner = (rank + p) % world;
            const int have = s_take[owner];
            for (int j = s_done[owner]; j < have; ++j)
                norm_received((size_t)owner * per + blockIdx.x + (size_t)j * G);
            data_sync();
            if (threadIdx.x == 0 && have > s_done[owner]) s_done[owner] = have;
        }
        data_sync();
    };

    RowLoads<NV, PEERS> ring[DEPTH];
    const int first = rank * per + blockIdx.x;
#pragma unroll
    for (int a = 0; a < DEPTH - 1; ++a)
        if (a < J) issue_row<NV, PEERS>(ring[a], x_mc, x_peer, residual, first + a * G, cols, nvec);
    for (int j = 0; j < J; ++j) {
        const int r = first + j * G;
        if (j + DEPTH - 1 < J)
            issue_row<NV, PEERS>(ring[DEPTH - 1], x_mc, x_peer, residual, r + (DEPTH - 1) * G, cols, nvec);
        const RowLoads<NV, PEERS>& cur = ring[0];
        float v[NV][8];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * kXThreads;
            if (c < nvec) {
                const size_t off = (size_t)r * cols + (size_t)c * 8;
                float x[8], t[8];
                unpack8(cur.x[i][0], x);
                if constexpr (PEERS > 1) {           // fp32 sum of the partials in rank order, rounded once
#pragma unroll
                    for (int p = 1; p < PEERS; ++p) {
                        float y[8];
                        unpack8(cur.x[i][p], y);
#pragma unroll
                        for (int e = 0; e < 8; ++e) x[e] += y[e];
                    }
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {     // what the switch hands back: the sum as bf16
                        const __nv_bfloat162 two = __floats2bfloat162_rn(x[e], x[e + 1]);
                        x[e] = __low2float(two);
                        x[e + 1] = __high2float(two);
                    }
                }
                unpack8(cur.t[i], t);
                uint4 packed;
                uint32_t* pw = &packed.x;
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const __nv_bfloat162 two = __floats2bfloat162_rn(x[e] + t[e], x[e + 1] + t[e + 1]);
                    pw[e / 2] = *reinterpret_cast<const uint32_t*>(&two);
                }
                if constexpr (SCATTER) {
                    *reinterpret_cast<uint4*>(sum_local + off) = packed;
                } else if constexpr (PEERS > 0) {
#pragma unroll
                    for (int p = 0; p < PEERS; ++p) *reinterpret_cast<uint4*>(sum_peer[p] + off) = packed;
                } else {
                    multimem_st_16(sum_mc + off, packed);
                }
                if constexpr (NORM) {
                    unpack8(packed, v[i]);                 // normalise the rounded sum, as a reader of `sum` would
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
                }
            }
        }
        if constexpr (!SCATTER) {
            __syncwarp();                                  // this warp's part of the row is on its way
            if (lane == 0) red_release_cta_shared_add(&s_warps_done, 1);
            // the counter reads "rows finished" only while no warp runs a row ahead of another: with the norm
            // the block reductions below keep the warps together, without it this barrier does
            if constexpr (!NORM) data_sync();
        }
        if constexpr (NORM) {
            const float inv = inv_rms(ss);
            store_norm<NV>(v, inv, w, norm_local + (size_t)r * cols, nvec);
            if (j + 1 < J) drain();
        }
#pragma unroll
        for (int a = 0; a + 1 < DEPTH; ++a) ring[a] = ring[a + 1];
    }

    if constexpr (SCATTER) {
        // every load of this warp has returned (its data was consumed): the closing flag may go out
        __syncwarp();
        if (lane == 0) red_release_cta_shared_add(&s_warps_done, 1);
    } else if constexpr (NORM) {
        // the rest of the other ranks' rows, owner by owner, row by row as the signalling warp publishes them
        for (int p = 1; p < world; ++p) {
            const int owner = (rank + p) % world;
            for (int j = s_done[owner]; j < J; ++j) {
                if (threadIdx.x == 0) {
                    for (uint32_t spin = 0; ld_acquire_cta_shared(&s_avail[owner]) <= j && spin < kCommSpinCap; ++spin)
                        if (spin > 16) __nanosleep(64);
                }
                data_sync();
                norm_received((size_t)owner * per + blockIdx.x + (size_t)j * G);
            }
        }
    }
    // (all-reduce without the norm: the signalling warp alone waits for the peers' last flags, which also
    // means that none of them still reads this rank's partial output; the kernel ends when it returns)
}

// The ranks meet: thread p tells rank p that this rank arrived for the `epoch`-th time and waits for
// rank p to say the same.  One CTA, bounded polls.
__global__ void rank_barrier_kernel(uint32_t* const* flags, uint32_t* launch_count, int rank, int world,
                                    int32_t* status) {
    __shared__ uint32_t s_epoch;
    if (threadIdx.x == 0) s_epoch = launch_count[0] + 1;
    __syncthreads();
    __threadfence_system();                        // work that preceded the barrier in this stream is visible first
    if ((int)threadIdx.x < world) {
        st_release_sys(flags[threadIdx.x] + rank, s_epoch);
        flag_wait(flags[rank] + threadIdx.x, s_epoch, status);
    }
    __syncthreads();
    if (threadIdx.x == 0) launch_count[0] = s_epoch;
}

}  // namespace ktk

using namespace ktk;

extern "C" int ktk_rank_barrier(const void* flag_ptrs, void* launch_count, int32_t rank, int32_t world,
                                int32_t* status, void* stream) {
    if (!flag_ptrs || !launch_count || world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world) {
        set_error("ktk_rank_barrier: bad arguments rank=%d world=%d", rank, world);
        return KTK_ERR_ARG;
    }
    rank_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t* const*)flag_ptrs, (uint32_t*)launch_count, rank,
                                                            world, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_rank_barrier");
    return KTK_OK;
}

// CTAs resident per SM: only the multicast form on rows of up to 4096 elements keeps few enough registers
// for two; the others hold more of a row (and more rows in flight) per thread and run one per SM
static int exchange_ctas_per_sm(int peers, int nv) { return (peers == 0 && nv == 1) ? 2 : 1; }

// Every CTA must be resident: same-index CTAs of the ranks wait for one another.
static int exchange_grid(int64_t rows, int world, int peers, int nv) {
    const int64_t per = rows / world;
    const int64_t cap = (int64_t)exchange_ctas_per_sm(peers, nv) * sm_count();
    return (int)(per < cap ? per : cap);
}

extern "C" int32_t ktk_exchange_grid(int64_t rows, int32_t world) {
    if (rows <= 0 || world <= 0 || rows % world != 0) return 0;
    return exchange_grid(rows, world, 0, 1);            // the largest grid any form launches
}

extern "C" int ktk_exchange_rows(const void* x_multicast, const void* x_peer_ptrs, const void* residual, const void* w,
                                 void* sum_multicast, const void* sum_peer_ptrs, void* out_local, void* norm_local,
                                 const void* flag_ptrs, void* launch_count, int32_t rank, int32_t world, int64_t rows,
                                 int32_t cols, float eps, int32_t mode, int32_t result, int32_t* status,
                                 void* stream) {
    if (world < 2 || world > kCommMaxWorld || rank < 0 || rank >= world || rows <= 0 || cols <= 0) {
        set_error("ktk_exchange_rows: bad arguments rank=%d world=%d rows=%lld cols=%d", rank, world, (long long)rows,
                  cols);
        return KTK_ERR_ARG;
    }
    if (mode != KTK_ALLREDUCE_AUTO && mode != KTK_ALLREDUCE_MULTICAST && mode != KTK_ALLREDUCE_PEER) {
        set_error("ktk_exchange_rows: unknown mode %d", mode);
        return KTK_ERR_ARG;
    }
    if (result != KTK_EXCHANGE_ALLREDUCE_NORM && result != KTK_EXCHANGE_ALLREDUCE && result != KTK_EXCHANGE_SCATTER) {
        set_error("ktk_exchange_rows: unknown result kind %d", result);
        return KTK_ERR_ARG;
    }
    const bool scatter = result == KTK_EXCHANGE_SCATTER;
    const bool norm = result == KTK_EXCHANGE_ALLREDUCE_NORM;
    const bool have_peer = x_peer_ptrs != nullptr && (scatter || sum_peer_ptrs != nullptr);
    const bool have_mc = x_multicast != nullptr && (scatter || sum_multicast != nullptr);
    if (mode == KTK_ALLREDUCE_AUTO)       // few ranks: a rank's own share would cross the switch and come back
        mode = (have_peer && (world == 2 || world == 4)) ? KTK_ALLREDUCE_PEER : KTK_ALLREDUCE_MULTICAST;
    if (mode == KTK_ALLREDUCE_PEER && world != 2 && world != 4) {
        set_error("ktk_exchange_rows: the peer-load form is built for 2 and 4 ranks (got %d)", world);
        return KTK_ERR_UNSUPPORTED;
    }
    if ((mode == KTK_ALLREDUCE_PEER && !have_peer) || (mode == KTK_ALLREDUCE_MULTICAST && !have_mc) || !residual ||
        !out_local || !flag_ptrs || !launch_count || (norm && (!w || !norm_local))) {
        set_error("ktk_exchange_rows: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (rows % world != 0 || cols % 8 != 0 || cols > 8 * kXThreads * kXMaxVec || rows > 2147483647LL) {
        set_error("ktk_exchange_rows: rows (%lld) must divide by the ranks (%d), cols (%d) by 8 and be <= %d",
                  (long long)rows, world, cols, 8 * kXThreads * kXMaxVec);
        return KTK_ERR_UNSUPPORTED;
    }
    const uintptr_t al = (uintptr_t)x_multicast | (uintptr_t)residual | (uintptr_t)w | (uintptr_t)sum_multicast |
                         (uintptr_t)out_local | (uintptr_t)norm_local;
    if ((al & 15u) != 0) { set_error("ktk_exchange_rows: pointers must be 16-byte aligned"); return KTK_ERR_ARG; }
    const int nv = (cols + 8 * kXThreads - 1) / (8 * kXThreads);
    const int peers = (mode == KTK_ALLREDUCE_PEER) ? world : 0;
    const int grid = exchange_grid(rows, world, peers, nv);
    // flag values of one launch: start, one per owned row, (scatter) end
    const uint32_t stride = (uint32_t)((rows / world + grid - 1) / grid + 2);
#define KTK_X_LAUNCH(NV, PEERS, SC, NO)                                                                        \
    exchange_rows_kernel<NV, PEERS, SC, NO><<<grid, kXAllThreads, 0, (cudaStream_t)stream>>>(                     \
        (const __nv_bfloat16*)x_multicast, (const __nv_bfloat16* const*)x_peer_ptrs,                           \
        (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)sum_multicast,                \
        (__nv_bfloat16* const*)sum_peer_ptrs, (__nv_bfloat16*)out_local, (__nv_bfloat16*)norm_local,           \
        (uint32_t* const*)flag_ptrs, (uint32_t*)launch_count, rank, world, (int)rows, cols, eps, stride, status)
#define KTK_X_KIND(NV, PEERS)                                                                                  \
    do {                                                                                                       \
        if (scatter) KTK_X_LAUNCH(NV, PEERS, true, false);                                                     \
        else if (norm) KTK_X_LAUNCH(NV, PEERS, false, true);                                                   \
        else KTK_X_LAUNCH(NV, PEERS, false, false);                                                            \
    } while (0)
#define KTK_X_NV(PEERS)                                                                                        \
    do {                                                                                                       \
        if (nv <= 1) KTK_X_KIND(1, PEERS);                                                                     \
        else KTK_X_KIND(2, PEERS);                                                                             \
    } while (0)
    if (peers == 0) KTK_X_NV(0);
    else if (peers == 2) KTK_X_NV(2);
    else KTK_X_NV(4);
#undef KTK_X_NV
#undef KTK_X_KIND
#undef KTK_X_LAUNCH
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_exchange_rows");
    return KTK_OK;
}
