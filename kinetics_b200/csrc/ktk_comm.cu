// o_proj all-reduce fused with the residual add and the post-attention RMSNorm,
// over NVSwitch multicast (multimem) instead of a separate NCCL all-reduce followed
// by an element-wise kernel.
//
// Every rank holds its partial o_proj output X_r [rows, cols] in a buffer that is mapped
// into one multicast object, and the residual (identical on all ranks).  Rank r owns the
// rows [r * rows / world, (r + 1) * rows / world):
//   1. barrier: every rank's X is complete (same-index CTAs of all ranks meet)
//   2. s = bf16( multimem.ld_reduce.add(X)[row] + residual[row] )   -- the switch adds the partials
//      multimem.st of s: every rank receives the row (the only bytes that cross NVLink twice)
//      n = s * rsqrt(mean(s^2) + eps) * w, from registers, into this rank's own `norm`
//   3. signal: this CTA's rows are on their way to every rank
//   4. owner by owner, as the same-index CTA of that rank signals: its rows of `sum` are normalised
//      locally (read from L2) into `norm`
// The barriers are flags in peer memory (one word per (CTA, source rank)), written with
// release and polled with acquire at system scope; the values grow from launch to launch
// (a per-CTA launch counter in local memory), so nothing needs resetting and the kernel can
// sit in a CUDA graph.  Every poll loop is bounded: on expiry the CTA records
// KTK_STATUS_TIMEOUT and goes on without waiting.
#include "ktk_comm.cuh"

namespace ktk {

// RMSNorm of one row held in registers (v, the bf16-rounded sum) -> plain stores to this rank's `norm`
template <int NV>
__device__ __forceinline__ void norm_row_store(const float (&v)[NV][8], float ss, float* part,
                                               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* norm_row,
                                               int nvec, int cols, float eps) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();                                   // `part` of the previous row has been read
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kCommThreads / 32; ++i) tot += part[i];
    const float inv = rsqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * kCommThreads;
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

// NV: vectors per thread, cols <= NV * 8 * kCommThreads.
// PEERS = 0: the switch reduces and multicasts (x_mc / sum_mc are multicast addresses).
// PEERS = world (2 or 4): plain peer loads and stores instead (x_peer / sum_peer hold every rank's
// buffer address): a rank's own data then stays off the links, which at 2 ranks is a third of the
// multicast form's traffic.
template <int NV, int PEERS>
__global__ void __launch_bounds__(kCommThreads, 4)
allreduce_add_rmsnorm_kernel(const __nv_bfloat16* x_mc, const __nv_bfloat16* const* x_peer,
                             const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                             __nv_bfloat16* sum_mc, __nv_bfloat16* const* sum_peer,
                             const __nv_bfloat16* sum_local, __nv_bfloat16* norm_local, uint32_t* const* flags,
                             uint32_t* launch_count, int rank, int world, int rows, int cols, float eps,
                             int32_t* status) {
    __shared__ float part[kCommThreads / 32];
    __shared__ uint32_t s_epoch;
    if (threadIdx.x == 0) s_epoch = launch_count[blockIdx.x];
    __syncthreads();
    const uint32_t epoch = s_epoch;

    cta_signal_all_ranks(flags, rank, world, 2 * epoch + 1);
    cta_wait_all_ranks(flags, rank, world, 2 * epoch + 1, status);        // every rank's partial output is complete

    const int per = rows / world;
    const int nvec = cols / 8;
    // the rows this rank owns: reduce through the switch, add the residual, multicast the sum,
    // normalise from registers
    for (int r = rank * per + blockIdx.x; r < (rank + 1) * per; r += gridDim.x) {
        float v[NV][8];
        float ss = 0.0f;
        constexpr int kSrc = PEERS > 0 ? PEERS : 1;
        uint4 xr[NV][kSrc], tr[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {          // all of the row's loads first
            const int c = threadIdx.x + i * kCommThreads;
            if (c < nvec) {
                const size_t off = (size_t)r * cols + (size_t)c * 8;
                if constexpr (PEERS > 0) {
#pragma unroll
                    for (int p = 0; p < PEERS; ++p) xr[i][p] = __ldcg(reinterpret_cast<const uint4*>(x_peer[p] + off));
                } else {
                    xr[i][0] = multimem_ld_reduce_bf16x8(x_mc + off);
                }
                tr[i] = __ldg(reinterpret_cast<const uint4*>(residual + off));
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * kCommThreads;
            if (c < nvec) {
                const size_t off = (size_t)r * cols + (size_t)c * 8;
                float x[8], t[8];
                unpack8(xr[i][0], x);
                if constexpr (PEERS > 1) {           // fp32 sum of the partials in rank order, rounded once
#pragma unroll
                    for (int p = 1; p < PEERS; ++p) {
                        float y[8];
                        unpack8(xr[i][p], y);
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
                unpack8(tr[i], t);
                uint4 packed;
                uint32_t* pw = &packed.x;
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const __nv_bfloat162 two = __floats2bfloat162_rn(x[e] + t[e], x[e + 1] + t[e + 1]);
                    pw[e / 2] = *reinterpret_cast<const uint32_t*>(&two);
                }
                if constexpr (PEERS > 0) {
#pragma unroll
                    for (int p = 0; p < PEERS; ++p) *reinterpret_cast<uint4*>(sum_peer[p] + off) = packed;
                } else {
                    multimem_st_16(sum_mc + off, packed);
                }
                unpack8(packed, v[i]);                     // normalise the rounded sum, as a reader of `sum` would
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
            }
        }
        norm_row_store<NV>(v, ss, part, w, norm_local + (size_t)r * cols, nvec, cols, eps);
    }
    __threadfence_system();                                // this CTA's rows are on their way to every rank
    cta_signal_all_ranks(flags, rank, world, 2 * epoch + 2);

    // the rows the same-index CTAs of the other ranks sent, one owner after another as its flag arrives:
    // normalise them from this rank's copy of `sum` (read at L2, where the peers' stores land).  Having
    // seen every peer's second flag also means that no peer still reads this rank's `x`.
    for (int p = 1; p < world; ++p) {
        const int owner = (rank + p) % world;
        cta_wait_rank(flags, rank, world, owner, 2 * epoch + 2, status);
        for (int r = owner * per + blockIdx.x; r < (owner + 1) * per; r += gridDim.x) {
            float v[NV][8];
            float ss = 0.0f;
            uint4 sr[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = threadIdx.x + i * kCommThreads;
                if (c < nvec) sr[i] = __ldcg(reinterpret_cast<const uint4*>(sum_local + (size_t)r * cols + (size_t)c * 8));
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = threadIdx.x + i * kCommThreads;
                if (c < nvec) {
                    unpack8(sr[i], v[i]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
                }
            }
            norm_row_store<NV>(v, ss, part, w, norm_local + (size_t)r * cols, nvec, cols, eps);
        }
    }
    if (threadIdx.x == 0) launch_count[blockIdx.x] = epoch + 1;
}

}  // namespace ktk

using namespace ktk;

extern "C" int32_t ktk_allreduce_grid(int64_t rows, int32_t world) {
    if (rows <= 0 || world <= 0) return 0;
    const int64_t per = rows / world;
    const int64_t cap = 4LL * sm_count();        // four 256-thread CTAs fit an SM: every CTA is resident
    return (int32_t)(per < cap ? per : cap);
}

extern "C" int ktk_allreduce_add_rmsnorm(const void* x_multicast, const void* x_peer_ptrs, const void* residual,
                                         const void* w, void* sum_multicast, const void* sum_peer_ptrs,
                                         const void* sum_local, void* norm_local, const void* flag_ptrs,
                                         void* launch_count, int32_t rank, int32_t world, int64_t rows,
                                         int32_t cols, float eps, int32_t mode, int32_t* status, void* stream) {
    if (world < 2 || world > kCommMaxWorld || rank < 0 || rank >= world || rows <= 0 || cols <= 0) {
        set_error("ktk_allreduce_add_rmsnorm: bad arguments rank=%d world=%d rows=%lld cols=%d", rank, world,
                  (long long)rows, cols);
        return KTK_ERR_ARG;
    }
    if (mode != KTK_ALLREDUCE_AUTO && mode != KTK_ALLREDUCE_MULTICAST && mode != KTK_ALLREDUCE_PEER) {
        set_error("ktk_allreduce_add_rmsnorm: unknown mode %d", mode);
        return KTK_ERR_ARG;
    }
    const bool have_peer = x_peer_ptrs != nullptr && sum_peer_ptrs != nullptr;
    const bool have_mc = x_multicast != nullptr && sum_multicast != nullptr;
    if (mode == KTK_ALLREDUCE_AUTO)       // few ranks: a rank's own share would cross the switch and come back
        mode = (have_peer && (world == 2 || world == 4)) ? KTK_ALLREDUCE_PEER : KTK_ALLREDUCE_MULTICAST;
    if (mode == KTK_ALLREDUCE_PEER && world != 2 && world != 4) {
        set_error("ktk_allreduce_add_rmsnorm: the peer-load form is built for 2 and 4 ranks (got %d)", world);
        return KTK_ERR_UNSUPPORTED;
    }
    if ((mode == KTK_ALLREDUCE_PEER && !have_peer) || (mode == KTK_ALLREDUCE_MULTICAST && !have_mc) || !residual ||
        !w || !sum_local || !norm_local || !flag_ptrs || !launch_count) {
        set_error("ktk_allreduce_add_rmsnorm: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (rows % world != 0 || cols % 8 != 0 || cols > 8 * kCommThreads * kCommMaxVec || rows > 2147483647LL) {
        set_error("ktk_allreduce_add_rmsnorm: rows (%lld) must divide by the ranks (%d), cols (%d) by 8 and be <= %d",
                  (long long)rows, world, cols, 8 * kCommThreads * kCommMaxVec);
        return KTK_ERR_UNSUPPORTED;
    }
    const uintptr_t al = (uintptr_t)x_multicast | (uintptr_t)residual | (uintptr_t)w | (uintptr_t)sum_multicast |
                         (uintptr_t)sum_local | (uintptr_t)norm_local;
    if ((al & 15u) != 0) { set_error("ktk_allreduce_add_rmsnorm: pointers must be 16-byte aligned"); return KTK_ERR_ARG; }
    const int grid = ktk_allreduce_grid(rows, world);
    const int nv = (cols + 8 * kCommThreads - 1) / (8 * kCommThreads);
    const int peers = (mode == KTK_ALLREDUCE_PEER) ? world : 0;
#define KTK_COMM_LAUNCH(NV, PEERS)                                                                            \
    allreduce_add_rmsnorm_kernel<NV, PEERS><<<grid, kCommThreads, 0, (cudaStream_t)stream>>>(                 \
        (const __nv_bfloat16*)x_multicast, (const __nv_bfloat16* const*)x_peer_ptrs,                          \
        (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)sum_multicast,               \
        (__nv_bfloat16* const*)sum_peer_ptrs, (const __nv_bfloat16*)sum_local, (__nv_bfloat16*)norm_local,    \
        (uint32_t* const*)flag_ptrs, (uint32_t*)launch_count, rank, world, (int)rows, cols, eps, status)
#define KTK_COMM_NV(PEERS)                                                                                    \
    do {                                                                                                      \
        if (nv <= 1) KTK_COMM_LAUNCH(1, PEERS);                                                               \
        else if (nv == 2) KTK_COMM_LAUNCH(2, PEERS);                                                          \
        else KTK_COMM_LAUNCH(4, PEERS);                                                                       \
    } while (0)
    if (peers == 0) KTK_COMM_NV(0);
    else if (peers == 2) KTK_COMM_NV(2);
    else KTK_COMM_NV(4);
#undef KTK_COMM_NV
#undef KTK_COMM_LAUNCH
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_allreduce_add_rmsnorm");
    return KTK_OK;
}
