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
// link (the sums the others send) are busy at the same time, and the local normalisation of the
// received rows hides behind the link time.  In the lock-step form of ktk_comm.cu all CTAs load,
// then all CTAs store, then all normalise.
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

// block-wide sum of squares -> 1 / rms
__device__ __forceinline__ float block_inv_rms(float ss, float* part, int cols, float eps) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();                                   // `part` of the previous row has been read
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kXThreads / 32; ++i) tot += part[i];
    return rsqrtf(tot / (float)cols + eps);
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

// RMSNorm of a row of this rank's own copy of `sum` (a row another rank sent), read at L2
template <int NV>
__device__ __forceinline__ void norm_received_row(const __nv_bfloat16* sum_row, const __nv_bfloat16* __restrict__ w,
                                                  __nv_bfloat16* norm_row, float* part, int nvec, int cols, float eps) {
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
    const float inv = block_inv_rms(ss, part, cols, eps);
    store_norm<NV>(v, inv, w, norm_row, nvec);
}

// NV: vectors per thread.  PEERS = 0: the switch reduces and multicasts; PEERS = world (2 or 4): peer
// loads and stores.  SCATTER: the sums of the owned rows stay on this rank (reduce-scatter), nothing
// is sent and nothing is normalised.  NORM (all-reduce form only): RMSNorm of every row into `norm`.
template <int NV, int PEERS, bool SCATTER, bool NORM>
__global__ void __launch_bounds__(kXThreads, (PEERS == 4 || NV == 2) ? 1 : 2)
exchange_rows_kernel(const __nv_bfloat16* x_mc, const __nv_bfloat16* const* x_peer,
                     const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* sum_mc, __nv_bfloat16* const* sum_peer, __nv_bfloat16* sum_local,
                     __nv_bfloat16* norm_local, uint32_t* const* flags, uint32_t* launch_count, int rank, int world,
                     int rows, int cols, float eps, uint32_t stride, int32_t* status) {
    __shared__ float part[kXThreads / 32];
    __shared__ uint32_t s_epoch;
    __shared__ int s_avail[kCommMaxWorld];      // rows the same-index CTA of rank p has flagged
    __shared__ int s_done[kCommMaxWorld];       // rows of rank p this CTA has normalised
    if (threadIdx.x == 0) s_epoch = launch_count[blockIdx.x];
    if (threadIdx.x < kCommMaxWorld) { s_avail[threadIdx.x] = 0; s_done[threadIdx.x] = 0; }
    __syncthreads();
    const uint32_t base = s_epoch * stride;
    const int G = gridDim.x;
    const int per = rows / world;
    const int nvec = cols / 8;
    const int J = (per - (int)blockIdx.x + G - 1) / G;      // rows of every owner that fall to CTAs of this index
    uint32_t* my_flags = flags[rank] + (size_t)blockIdx.x * world;

    // every rank's partial output is complete (its GEMM precedes this kernel in stream order)
    if ((int)threadIdx.x < world) st_release_sys(flags[threadIdx.x] + (size_t)blockIdx.x * world + rank, base + 1);
    if ((int)threadIdx.x < world) flag_wait(my_flags + threadIdx.x, base + 1, status);
    __syncthreads();

    // rows another rank has flagged so far: normalise those not yet done (never blocks)
    auto drain = [&]() {
        if ((int)threadIdx.x < world) {
            const int32_t got = (int32_t)(ld_acquire_sys(my_flags + threadIdx.x) - (base + 1));
            s_avail[threadIdx.x] = got < 0 ? 0 : (got > J ? J : got);
        }
        __syncthreads();
        for (int p = 1; p < world; ++p) {
            const int owner = (rank + p) % world;
            const int have = s_avail[owner];
            for (int j = s_done[owner]; j < have; ++j) {
                const size_t r = (size_t)owner * per + blockIdx.x + (size_t)j * G;
                norm_received_row<NV>(sum_local + r * cols, w, norm_local + r * cols, part, nvec, cols, eps);
            }
            __syncthreads();
            if (threadIdx.x == 0 && have > s_done[owner]) s_done[owner] = have;
        }
        __syncthreads();
    };

    RowLoads<NV, PEERS> cur, nxt;
    const int first = rank * per + blockIdx.x;
    if (J > 0) issue_row<NV, PEERS>(cur, x_mc, x_peer, residual, first, cols, nvec);
    for (int j = 0; j < J; ++j) {
        const int r = first + j * G;
        if (j + 1 < J) issue_row<NV, PEERS>(nxt, x_mc, x_peer, residual, r + G, cols, nvec);
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
            __threadfence_system();                        // this row is on its way to every rank
            __syncthreads();
            if ((int)threadIdx.x < world)
                st_release_sys(flags[threadIdx.x] + (size_t)blockIdx.x * world + rank, base + 2 + j);
        }
        if constexpr (NORM) {
            const float inv = block_inv_rms(ss, part, cols, eps);
            store_norm<NV>(v, inv, w, norm_local + (size_t)r * cols, nvec);
            if (j + 1 < J) drain();
        }
        if (j + 1 < J) cur = nxt;
    }

    if constexpr (SCATTER) {
        // nobody may overwrite its partial output while a peer still reads it: meet once more
        __syncthreads();
        if ((int)threadIdx.x < world) st_release_sys(flags[threadIdx.x] + (size_t)blockIdx.x * world + rank, base + 2);
        if ((int)threadIdx.x < world) flag_wait(my_flags + threadIdx.x, base + 2, status);
    } else {
        // the rest of the other ranks' rows, owner by owner, row by row as the flags arrive.  Having
        // seen a peer's last flag also means that it no longer reads this rank's partial output.
        for (int p = 1; p < world; ++p) {
            const int owner = (rank + p) % world;
            if constexpr (NORM) {
                for (int j = s_done[owner]; j < J; ++j) {
                    if (threadIdx.x == 0) flag_wait(my_flags + owner, base + 2 + j, status);
                    __syncthreads();
                    const size_t r = (size_t)owner * per + blockIdx.x + (size_t)j * G;
                    norm_received_row<NV>(sum_local + r * cols, w, norm_local + r * cols, part, nvec, cols, eps);
                }
            } else {
                if (threadIdx.x == 0) flag_wait(my_flags + owner, base + 1 + J, status);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) launch_count[blockIdx.x] = s_epoch + 1;
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

// 512-thread CTAs resident per SM: the peer form at 4 ranks and rows wider than 4096 elements hold
// more of a row per thread and run one per SM
static int exchange_ctas_per_sm(int peers, int nv) { return (peers == 4 || nv == 2) ? 1 : 2; }

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
    exchange_rows_kernel<NV, PEERS, SC, NO><<<grid, kXThreads, 0, (cudaStream_t)stream>>>(                     \
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
