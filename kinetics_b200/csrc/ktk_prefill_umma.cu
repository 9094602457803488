// Causal prefill attention over the paged KV cache on the fifth-generation tensor cores (tcgen05, accumulators
// in tensor memory).  Same contract as prefill_mma_kernel (ktk_prefill.cu); replaces
// flashinfer.single_prefill_with_kv_cache of LiteSys/litesys/attention/batch_cache.py:129-145.
//
// One CTA per (sequence, kv head, tile of 128 / G new tokens): the 128 rows of the tile are the (token, head of
// the query group) pairs; row r belongs to softmax thread r and lives in lane r of tensor memory.  The history is
// walked in blocks of 64 keys (four pages).  Roles:
//     issuing warp (one lane)   TMA: K and V of a block -> shared memory, 16-row x 128-byte boxes under the
//                               128-byte swizzle, which is the operand layout tcgen05.mma reads; K two blocks
//                               ahead, V one.
//                               S[128 x 64]   = Q[128 x 128] . K^T    8 x tcgen05.mma (M 128, N 64, K 16), D in TMEM
//                               O[128 x 128] += P[128 x 64] . V       4 x tcgen05.mma (M 128, N 128, K 16), A = P
//                               from tensor memory, B = V read MN-major: the page rows as they lie
//                               S of block j + 1 is issued before O += P.V of block j: the tensor cores work on it
//                               while the threads do the softmax of block j.
//     softmax thread r          row r of S <- tcgen05.ld; scale, causal / fill-level mask, running max and sum;
//                               P = 2^(S - reference) as bf16 pairs back over the first 32 columns of that S
//                               (tcgen05.st); the O row in tensor memory rescaled when the reference moved
// and at the end row r of O is read back, divided by the row sum and stored.  tcgen05.commit -> mbarrier tells
// the threads when S and O are complete; the softmax warps meet at one named barrier per block and one of them
// then tells the issuing warp that P is in place.  Two CTAs per SM (97 KiB of shared memory, 256 TMEM columns
// each).  Every wait is bounded; tensor memory is released on every path.
#include "ktk_decode_mma.cuh"
#include "ktk_prefill_umma.cuh"

namespace ktk {

constexpr int kUmRows = 128;                 // rows of a tile = softmax threads of a CTA
constexpr int kUmThreads = kUmRows + 64;     // + the warp that feeds the tensor cores + the warp that issues the copies
constexpr int kUmKeys = 64;                  // keys per block
constexpr int kUmPagesPerBlock = kUmKeys / kPageSize;
constexpr int kUmTmemCols = 256;             // S of two blocks: columns [0, 64) and [64, 128); O: [128, 256)
constexpr int kUmColS = 0, kUmColO = 128;
constexpr int kUmQBytes = 2 * kUmRows * 128; // two tiles of [128 rows][64 dims]
constexpr int kUmKBytes = 2 * kUmKeys * 128; // two tiles of [64 keys][64 dims]
constexpr int kUmPBytes = kUmRows * 128;     // [128 rows][64 keys]: laid over the K tiles of its block (dead by then)
static_assert(kUmPBytes <= kUmKBytes, "P reuses the K buffer");
constexpr int kUmSmem = kUmQBytes + 4 * kUmKBytes + 1024;     // Q | K, V of two blocks in flight

// ---- tcgen05 wrappers -------------------------------------------------------------------------------------
// shared-memory operand descriptor: start address, leading / stride byte offsets (all >> 4), version 1,
// 128-byte swizzle
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// instruction descriptor of kind::f16: fp32 accumulate, bf16 A and B, A K-major, M = 128
__device__ __forceinline__ uint32_t umma_idesc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(kUmRows >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (lane = row, two bf16 per column)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive fp32 columns of this thread's TMEM lane: both loads in flight before the one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&lo)[32], float (&hi)[32]) {
    uint32_t r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr), "r"(taddr + 32));
#pragma unroll
    for (int i = 0; i < 32; ++i) { lo[i] = __uint_as_float(r[i]); hi[i] = __uint_as_float(r[32 + i]); }
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
          "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
          "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
          "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
          "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
          "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st32_u32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Bounded wait without a suspend-time hint: the barriers of this kernel complete within microseconds, and the
// waiter should see that at once.  Gives up like mbar_wait (and raises *abort) after about a second of polling.
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile int* abort) {
    for (uint32_t i = 0; i < (1u << 24); ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 63u) == 63u && *abort) return false;
    }
    *abort = 1;
    return false;
}

// 2^x on the special-function unit (-inf -> 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` in a [rows][128 B] tile under the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// barrier of the softmax warps (named barrier 1); returns whether any of them raised `flag`
__device__ __forceinline__ bool softmax_sync_or(bool flag) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out) : "r"((uint32_t)flag), "n"(kUmRows) : "memory");
    return out != 0;
}

__global__ void __launch_bounds__(kUmThreads, 2)
prefill_umma_kernel(const PrefillUmmaParams p, const __grid_constant__ CUtensorMap kv_map) {
    extern __shared__ uint8_t um_raw[];
    // S complete (per S buffer) | K, V landed (per buffer) | P in place | O += P.V of a block complete = its V buffer
    // read out (per buffer)
    // (per-buffer barriers for the TMA warp: a barrier it waits on cannot run two phases ahead of it, because the next
    // phase needs the very copy it is about to issue)
    __shared__ __align__(8) uint64_t bar_s[2], bar_k[2], bar_v[2], bar_p, bar_vfree[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int kpos[2][kUmKeys];              // position of the key in row c of the block (INT_MAX: none)
    __shared__ int abort_flag;

    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(um_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = sm;
    uint8_t* sKV = sQ + kUmQBytes;                // [buffer][K | V]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool issuer = warp == kUmRows / 32;     // the fifth warp: tensor-core instructions (and TMEM allocation)
    const bool loader = warp == kUmRows / 32 + 1; // the sixth warp: TMA
    const int b = blockIdx.z, h = blockIdx.y;
    const int G = p.G, Hq = p.Hkv * G;
    const int tpc = kUmRows / G;                    // new tokens per CTA
    const int q0 = p.q_indptr[b];
    const int n_new = p.q_indptr[b + 1] - q0;
    // tiles late in a sequence see the longest history: they are launched first
    const int tok0 = (int)(gridDim.x - 1 - blockIdx.x) * tpc;
    if (tok0 >= n_new) return;                      // uniform for the CTA: nothing allocated yet

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
    const int n_blocks = (n_need + kUmPagesPerBlock - 1) / kUmPagesPerBlock;

    // a softmax thread's row
    const int my_tok = tok0 + tid / G, my_head = h * G + tid % G;
    const bool row_on = warp < kUmRows / 32 && my_tok < n_new;
    const int vis = row_on ? base_pos + my_tok + 1 : 0;     // keys at positions < vis are seen

    // tokens held by logical page e, and whether block `blk` has rows without a key (a page past the needed ones
    // or a page that is not full): those rows of V are cleared before use and the block is masked
    auto page_tokens = [&](int e) { return e == sp.n_pages - 1 ? sp.last_fill : (e == 0 ? sp.first_fill : kPageSize); };
    auto block_has_holes = [&](int blk) {
        const int e0 = blk * kUmPagesPerBlock, e1 = e0 + kUmPagesPerBlock - 1;
        if (e1 >= n_need) return true;
        if (e0 == 0 && sp.first_fill != kPageSize) return true;
        return e1 == sp.n_pages - 1 && sp.last_fill != kPageSize;
    };
    // positions of the keys of block `blk` (softmax threads 0..63, one row each)
    auto note_positions = [&](int blk) {
        if (blk >= n_blocks || tid >= kUmKeys) return;
        const int e = blk * kUmPagesPerBlock + (tid >> 4), slot = tid & 15;
        kpos[blk & 1][tid] = (e < n_need && slot < page_tokens(e)) ? page_first_pos(e, sp.first_fill) + slot : 0x7fffffff;
    };

    if (tid == 0) {
        mbar_init(&bar_s[0], 1);
        mbar_init(&bar_s[1], 1);
        mbar_init(&bar_p, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&bar_k[i], 1); mbar_init(&bar_v[i], 1); mbar_init(&bar_vfree[i], 1); }
        abort_flag = 0;
        mbar_init_fence();
    }
    if (warp < kUmRows / 32) {
        // Q row -> two swizzled tiles (zeros for rows past the last new token)
        const uint4* src = reinterpret_cast<const uint4*>(
            (const __nv_bfloat16*)p.q + ((int64_t)(q0 + (row_on ? my_tok : 0)) * Hq + my_head) * kHeadDim);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            const uint4 v = row_on ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(sQ + (c >> 3) * (kUmRows * 128) + swz(tid, c & 7)) = v;
        }
        note_positions(0);
        fence_proxy_async();
    } else if (issuer) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(kUmTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    bool alive = true;

    if (issuer) {
        if (lane == 0 && n_blocks > 0) {
            const uint32_t idesc_s = umma_idesc(kUmKeys, false);
            const uint32_t idesc_o = umma_idesc(kHeadDim, true);
            // S of block `blk` = Q . K^T into S buffer blk & 1, once its K has landed
            auto issue_s = [&](int blk) {
                const int buf = blk & 1;
                const uint32_t kaddr = smem_u32(sKV + buf * (2 * kUmKBytes));
                if (!mbar_wait_fast(&bar_k[buf], (blk >> 1) & 1, &abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int s = 0; s < kHeadDim / 16; ++s) {
                    const uint64_t a = umma_desc(smem_u32(sQ) + (s >> 2) * (kUmRows * 128) + (s & 3) * 32, 0, 1024);
                    const uint64_t bd = umma_desc(kaddr + (s >> 2) * (kUmKeys * 128) + (s & 3) * 32, 0, 1024);
                    umma_f16(tmem + kUmColS + buf * kUmKeys, a, bd, idesc_s, s > 0 ? 1u : 0u);
                }
                umma_commit(&bar_s[buf]);
                return true;
            };
            bool ok = issue_s(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int buf = j & 1;
                // S of the next block first: its S buffer was read out, and the P in it consumed, a block ago
                if (j + 1 < n_blocks) ok = issue_s(j + 1);
                // O += P . V once P is in place and V has landed
                ok = ok && mbar_wait_fast(&bar_p, j & 1, &abort_flag) && mbar_wait_fast(&bar_v[buf], (j >> 1) & 1, &abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t vaddr = smem_u32(sKV + buf * (2 * kUmKBytes) + kUmKBytes);
                const uint32_t s_col = kUmColS + buf * kUmKeys;
#pragma unroll
                for (int s = 0; s < kUmKeys / 16; ++s) {
                    const uint64_t bd = umma_desc(vaddr + s * (16 * 128), kUmVLbo, kUmVSbo);
                    umma_f16_ts(tmem + kUmColO, tmem + s_col + s * 8, bd, idesc_o, (j > 0 || s > 0) ? 1u : 0u);
                }
                umma_commit(&bar_vfree[buf]);
            }
        }
    } else if (loader) {
        if (lane == 0 && n_blocks > 0) {
            // K (which = 0) or V (which = 1) of block `blk` -> its buffer blk & 1: per page two boxes of 16 rows x 128 B
            auto issue_tma = [&](int blk, int which) {
                if (blk >= n_blocks) return;
                const int buf = blk & 1;
                uint64_t* bar = which ? &bar_v[buf] : &bar_k[buf];
                uint8_t* dst = sKV + buf * (2 * kUmKBytes) + which * kUmKBytes;
                int64_t pages[kUmPagesPerBlock];
                uint32_t bytes = 0;
#pragma unroll
                for (int pi = 0; pi < kUmPagesPerBlock; ++pi) {
                    const int e = blk * kUmPagesPerBlock + pi;
                    pages[pi] = -1;
                    if (e < n_need) {
                        const int64_t pg = p.kv_indices[sp.start + e];
                        if (pg < 0 || pg >= p.num_pages) {
                            if (which == 0) report(p.status, KTK_STATUS_BAD_PAGE);
                        } else {
                            pages[pi] = pg;
                            bytes += 2u * kPageSize * 128u;
                        }
                    }
                }
                if (bytes) mbar_arrive_expect_tx(bar, bytes);
                else mbar_arrive(bar);
#pragma unroll
                for (int pi = 0; pi < kUmPagesPerBlock; ++pi) {
                    if (pages[pi] < 0) continue;
                    const int z = (int)(pages[pi] * (2 * kPageSize)) + which * kPageSize;    // token row of slot 0
                    tma_load_3d(dst + pi * (kPageSize * 128), &kv_map, bar, 0, h, z);
                    tma_load_3d(dst + kUmKeys * 128 + pi * (kPageSize * 128), &kv_map, bar, 64, h, z);
                }
            };
            prefetch_tensormap(&kv_map);
            issue_tma(0, 0);
            issue_tma(1, 0);
            issue_tma(0, 1);
            for (int j = 0; j < n_blocks; ++j) {
                // K of block j + 2 goes over K of block j once S of block j is complete
                if (j + 2 < n_blocks) {
                    if (!mbar_wait_fast(&bar_s[j & 1], (j >> 1) & 1, &abort_flag)) break;
                    issue_tma(j + 2, 0);
                }
                // V of block j + 1 goes over V of block j - 1 once O += P.V of block j - 1 is complete
                if (j + 1 < n_blocks) {
                    if (j > 0 && !mbar_wait_fast(&bar_vfree[(j + 1) & 1], ((j - 1) >> 1) & 1, &abort_flag)) break;
                    issue_tma(j + 1, 1);
                }
            }
        }
    } else {
        const uint32_t my_tmem = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 lanes
        float m_run = -INFINITY, m_ref = 0.0f, l_run = 0.0f;   // running max, reference of the exponentials, row sum
        const int tile_min_vis = base_pos + tok0 + 1;
        for (int j = 0; j < n_blocks; ++j) {
            const int buf = j & 1;
            const uint32_t s_col = kUmColS + buf * kUmKeys;
            const bool holes = block_has_holes(j);
            // every row of the tile sees the whole block: no mask
            const bool clean = !holes && page_first_pos(j * kUmPagesPerBlock + kUmPagesPerBlock - 1, sp.first_fill) +
                                                 kPageSize <= tile_min_vis;
            if (!mbar_wait_fast(&bar_s[buf], (j >> 1) & 1, &abort_flag)) alive = false;
            tc_fence_after();

            float alpha = 1.0f;
            uint32_t packed[32];
            {
                float s_lo[32], s_hi[32];
                tmem_ld64(my_tmem + s_col, s_lo, s_hi);
                // masked columns become -inf; the scale (positive) is applied inside the exponent below
                if (!clean) {                       // uniform for the CTA
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        s_lo[c] = kpos[buf][c] < vis ? s_lo[c] : -INFINITY;
                        s_hi[c] = kpos[buf][32 + c] < vis ? s_hi[c] : -INFINITY;
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    mx0 = fmaxf(mx0, s_lo[c]);
                    mx1 = fmaxf(mx1, s_lo[c + 1]);
                    mx2 = fmaxf(mx2, s_hi[c]);
                    mx3 = fmaxf(mx3, s_hi[c + 1]);
                }
                const float mx = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
                // The reference point of the exponentials follows the running maximum only when that moved by
                // more than 2^8: P then stays below 256 (exact in fp32, fine in bf16) and the O row in tensor
                // memory is rescaled rarely instead of at almost every block.  The final division by the row sum,
                // taken against the same reference point, makes the result independent of it.
                float m_use;
                if (mx == -INFINITY) m_use = 0.0f;                     // a row that has seen nothing yet
                else if (m_run == -INFINITY || mx - m_ref > 8.0f) m_use = mx;
                else m_use = m_ref;
                alpha = (m_run == -INFINITY) ? 0.0f : exp2f(m_ref - m_use);
                m_ref = m_use;
                float sum = 0.0f;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p0 = ex2(fmaf(s_lo[2 * c], p.scale_log2, -m_use));
                    const float p1 = ex2(fmaf(s_lo[2 * c + 1], p.scale_log2, -m_use));
                    const float p2 = ex2(fmaf(s_hi[2 * c], p.scale_log2, -m_use));
                    const float p3 = ex2(fmaf(s_hi[2 * c + 1], p.scale_log2, -m_use));
                    sum += (p0 + p1) + (p2 + p3);
                    packed[c] = pack_bf16(p0, p1);      // keys 2c, 2c + 1 -> column c of P
                    packed[16 + c] = pack_bf16(p2, p3); // keys 32 + 2c, 33 + 2c -> column 16 + c
                }
                l_run = l_run * alpha + sum;
                m_run = mx;
            }
            // ---- the O row is rescaled only when the reference moved, and only then does this warp have to know
            //      that O += P.V of the previous block is over (per-buffer barrier: it cannot run ahead of us) ----
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {     // warp-uniform: tcgen05.ld / st are warp-wide
                if (!mbar_wait_fast(&bar_vfree[(j - 1) & 1], ((j - 1) >> 1) & 1, &abort_flag)) alive = false;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < kHeadDim; c += 32) {
                    float o[32];
                    tmem_ld32(my_tmem + kUmColO + c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    tmem_st32(my_tmem + kUmColO + c, o);
                }
            }
            // P as bf16 pairs over the first 32 columns of this block's S (read into registers above)
            tmem_st32_u32(my_tmem + s_col, packed);
            tmem_st_wait();
            if (holes) {                            // uniform: clear the rows of V that hold no key
                if (tid < kUmKeys && kpos[buf][tid] == 0x7fffffff) {
                    if (!mbar_wait_fast(&bar_v[buf], (j >> 1) & 1, &abort_flag)) alive = false;
                    uint8_t* vrow = sKV + buf * (2 * kUmKBytes) + kUmKBytes;
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        *reinterpret_cast<uint4*>(vrow + (c >> 3) * (kUmKeys * 128) + swz(tid, c & 7)) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async();
            }
            note_positions(j + 1);                  // kpos of the other buffer: block j - 1 is done with it
            tc_fence_before();
            // all rows of P in place, V cleared, positions written -- or, for all alike, a wait that ran out
            if (softmax_sync_or(!alive || abort_flag != 0)) { alive = false; break; }
            if (tid == 0) mbar_arrive(&bar_p);
        }
        if (alive && n_blocks > 0) {
            if (!mbar_wait_fast(&bar_vfree[(n_blocks - 1) & 1], ((n_blocks - 1) >> 1) & 1, &abort_flag)) alive = false;
            tc_fence_after();
        }
        if (alive) {
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            __nv_bfloat16* dst = (__nv_bfloat16*)p.o + ((int64_t)(q0 + (row_on ? my_tok : 0)) * Hq + my_head) * kHeadDim;
#pragma unroll
            for (int c = 0; c < kHeadDim; c += 32) {
                float o[32];
                if (n_blocks > 0) {                     // uniform for the CTA (the loads are warp-wide)
                    tmem_ld32(my_tmem + kUmColO + c, o);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0.0f;
                }
                if (row_on) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        v.x = pack_bf16(o[i] * inv, o[i + 1] * inv);
                        v.y = pack_bf16(o[i + 2] * inv, o[i + 3] * inv);
                        v.z = pack_bf16(o[i + 4] * inv, o[i + 5] * inv);
                        v.w = pack_bf16(o[i + 6] * inv, o[i + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (abort_flag && tid == 0) report(p.status, KTK_STATUS_TIMEOUT);
    if (issuer) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kUmTmemCols) : "memory");
    }
}

int launch_prefill_umma(const PrefillUmmaParams& p, int max_new_tokens, cudaStream_t st) {
    KTK_CUDA_TRY(cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kUmSmem),
                 "ktk_prefill_attention");
    const int tpc = kUmRows / p.G;
    const dim3 grid((unsigned)((max_new_tokens + tpc - 1) / tpc), (unsigned)p.Hkv, (unsigned)p.batch);
    DecodeParams d{};                               // only what the tensor map needs
    d.cache = p.cache; d.Hkv = p.Hkv; d.num_pages = p.num_pages;
    CUtensorMap map;
    const int rc = make_kv_tensor_map(&map, d);
    if (rc != KTK_OK) return rc;
    prefill_umma_kernel<<<grid, kUmThreads, kUmSmem, st>>>(p, map);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_prefill_attention");
    return KTK_OK;
}

}  // namespace ktk
