// What the two tensor-core decode kernels share: the shared-memory stage layout, the
// per-page tensor-core step and the tensor map over the KV cache.
#pragma once

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

// byte offset of 16-byte chunk `c16` (0..15 across the 256-byte row) of token row `tok`
// inside a K or V tile stored as two 128-byte-swizzled half tiles
__device__ __forceinline__ uint32_t tile_off(int tok, int c16) {
    return (uint32_t)((c16 >> 3) * kHalfTile + tok * 128 + (((c16 & 7) ^ (tok & 7)) << 4));
}

// A consumer warp's running softmax state for the two heads 2*tig, 2*tig+1 it holds
// (log2 domain) and its un-normalised O^T accumulators.
struct MmaState {
    float m0, m1, l0, l1;
    float acc[8][4];
    __device__ __forceinline__ void reset() {
        m0 = -INFINITY; m1 = -INFINITY; l0 = 0.0f; l1 = 0.0f;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    }
};

// Q^T fragments of the group of kv head h of sequence b: head gid, elements 16*ks + 2*tig (+8);
// heads past the group are zero
__device__ __forceinline__ void load_q_frags(uint32_t (&qb)[8][2], const void* q, int64_t first_head, int G,
                                             int lane) {
    const int gid = lane >> 2, tig = lane & 3;
    const uint32_t* qp = reinterpret_cast<const uint32_t*>((const __nv_bfloat16*)q + (first_head + gid) * kHeadDim);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        qb[ks][0] = (gid < G) ? __ldg(qp + ks * 8 + tig) : 0u;
        qb[ks][1] = (gid < G) ? __ldg(qp + ks * 8 + 4 + tig) : 0u;
    }
}

// One page on the tensor cores, by one warp.  `stage` is the generic address of the 8 KiB stage
// (K tile, then V tile, each as two swizzled half tiles), `ntok` the tokens the page holds.
//     S^T[16 tok x 8 heads]  = K[16 x 128] . Q^T          8 x mma.m16n8k16
//     O^T[128 x 8 heads]    += V^T[128 x 16] . P^T        8 x mma.m16n8k16
// CAUSAL (prefill): the 8 columns are (query token, head) pairs with their own horizon -- column 2*tig sees
// the first lim0 tokens of the page, column 2*tig+1 the first lim1 (both <= ntok, possibly 0).
template <bool CAUSAL>
__device__ __forceinline__ void mma_consume_page_t(MmaState& st, uint8_t* stage, int ntok,
                                                   const uint32_t (&qb)[8][2], float scale_log2, int lane,
                                                   int lim0, int lim1) {
    const int gid = lane >> 2;
    // per-lane ldmatrix row addresses (relative to the tile): lane supplies row (lane & 7) of matrix lane >> 3
    const int mj = lane >> 3, mr = lane & 7;
    const int k_tok = mr + 8 * (mj & 1), k_c = mj >> 1;     // K:  matrices (tok 0-7 | 8-15) x (chunk 2ks | 2ks+1)
    const int v_tok = mr + 8 * (mj >> 1), v_c = mj & 1;     // V^T: matrices (chunk 2mt | 2mt+1) x (tok 0-7 | 8-15)
    const uint32_t kt = smem_u32(stage);
    const uint32_t vt = kt + 2 * kHalfTile;
    if (ntok < kPageSize) {
        // rows past the fill level may hold anything: clear them in V so that 0 * x stays 0
        uint8_t* vrow = stage + 2 * kHalfTile;
        for (int c = lane; c < (kPageSize - ntok) * 16; c += 32) {
            const int t = ntok + (c >> 4), cc = c & 15;
            *reinterpret_cast<uint4*>(vrow + (cc >> 3) * kHalfTile + t * 128 + ((cc & 7) << 4)) = make_uint4(0, 0, 0, 0);
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
    float s00 = (s_a[0] + s_b[0]) * scale_log2, s01 = (s_a[1] + s_b[1]) * scale_log2;
    float s10 = (s_a[2] + s_b[2]) * scale_log2, s11 = (s_a[3] + s_b[3]) * scale_log2;
    if constexpr (CAUSAL) {
        if (gid >= lim0) s00 = -INFINITY;
        if (gid >= lim1) s01 = -INFINITY;
        if (gid + 8 >= lim0) s10 = -INFINITY;
        if (gid + 8 >= lim1) s11 = -INFINITY;
    } else {
        if (gid >= ntok) { s00 = -INFINITY; s01 = -INFINITY; }
        if (gid + 8 >= ntok) { s10 = -INFINITY; s11 = -INFINITY; }
    }
    float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);   // decode: finite, token 0 is valid
    // a column that has seen nothing yet and sees nothing here keeps m = -inf: subtract 0 instead of it
    const float b0 = (CAUSAL && mn0 == -INFINITY) ? 0.0f : mn0;
    const float b1 = (CAUSAL && mn1 == -INFINITY) ? 0.0f : mn1;
    const float al0 = exp2f(st.m0 - b0), al1 = exp2f(st.m1 - b1);
    // probabilities, rounded to bf16 once so that the normaliser matches what multiplies V
    const uint32_t p_lo = pack_bf16(exp2f(s00 - b0), exp2f(s01 - b1));   // tokens 0-7
    const uint32_t p_hi = pack_bf16(exp2f(s10 - b0), exp2f(s11 - b1));   // tokens 8-15
    float sum0 = __uint_as_float(p_lo << 16) + __uint_as_float(p_hi << 16);
    float sum1 = __uint_as_float(p_lo & 0xffff0000u) + __uint_as_float(p_hi & 0xffff0000u);
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, off);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, off);
    }
    st.m0 = mn0; st.m1 = mn1;
    st.l0 = st.l0 * al0 + sum0;
    st.l1 = st.l1 * al1 + sum1;
    // P^T as the B operand: transpose the two 8x8 (token x head) blocks
    const uint32_t pb0 = movmatrix_trans(p_lo);
    const uint32_t pb1 = movmatrix_trans(p_hi);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        uint32_t va[4];
        ldmatrix_x4_trans(va, vt + tile_off(v_tok, 2 * mt + v_c));
        st.acc[mt][0] *= al0; st.acc[mt][1] *= al1; st.acc[mt][2] *= al0; st.acc[mt][3] *= al1;
        mma_bf16(st.acc[mt], va, pb0, pb1);
    }
    if (ntok < kPageSize) fence_proxy_async();   // the cleared rows were written by ordinary stores
}

__device__ __forceinline__ void mma_consume_page(MmaState& st, uint8_t* stage, int ntok,
                                                 const uint32_t (&qb)[8][2], float scale_log2, int lane) {
    mma_consume_page_t<false>(st, stage, ntok, qb, scale_log2, lane, ntok, ntok);
}

// The four TMA tile loads of one page (K and V, each as two 16-row x 128-byte boxes) into a stage.
__device__ __forceinline__ void tma_load_page(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int64_t page,
                                              int h) {
    const int y = (int)(page * (2 * kPageSize));      // token row of K slot 0
    mbar_arrive_expect_tx(bar, kStageBytes);
    tma_load_3d(dst, map, bar, 0, h, y);
    tma_load_3d(dst + kHalfTile, map, bar, 64, h, y);
    tma_load_3d(dst + 2 * kHalfTile, map, bar, 0, h, y + kPageSize);
    tma_load_3d(dst + 3 * kHalfTile, map, bar, 64, h, y + kPageSize);
}

// Tensor map over the cache seen as [token rows = pages*2*16][Hkv][128], innermost first, in boxes of
// 16 rows x 64 elements with the 128-byte swizzle.
int make_kv_tensor_map(CUtensorMap* map, const DecodeParams& p);

int launch_decode_stream(const DecodeParams& p, int G, int max_entries, cudaStream_t st);
int stream_grid(int64_t units, int max_entries);
size_t stream_workspace_bytes(int G);

}  // namespace ktk
