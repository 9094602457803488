// The LiteSys decode chain function by function, on its own cache layout: an unpaged
// [max_batch, Hkv, max_len, D] key cache and value cache, an fp32 logits buffer
// [rows, Hq, max_len] that the steps hand to one another.
//
//   ktk_copy_to_cache   copy_to_cache            LiteSys/litesys/attention/cache_utils.py:5-51
//   ktk_qk              qk                       cache_utils.py:54-93, :173-190
//   ktk_block_topk_mask blockwise_topk_sparsity  sparsity_utils.py:24-47
//   ktk_softmax_rows    softmax                  cache_utils.py:97-130, :216-226
//   ktk_sv              sv                       cache_utils.py:135-169, :193-212
//
// They exist so that code written against those functions runs unchanged; they read every key
// and value of a sequence, which is what the paged block top-k kernels avoid (ktk_select_v +
// ktk_sparse_decode_v compute the same result from the selected pages only).
//
// Like the reference kernels, ktk_qk / ktk_softmax_rows / ktk_sv take `offset` indexed by the ROW
// of the active batch (cache_utils.py:67,106,149) while the cache slot comes from batch_idx[row].
#include "ktk_common.cuh"

namespace ktk {

constexpr int kChainThreads = 256;

// One (row, kv head): the new key of the row goes to cache[batch_id[row], h, offset[row], :].
template <typename T>
__global__ void copy_to_cache_kernel(T* __restrict__ cache, const T* __restrict__ src,
                                     const int64_t* __restrict__ batch_id, const int32_t* __restrict__ offset,
                                     int Hkv, int64_t max_batch, int64_t max_len, int64_t src_row_stride,
                                     int64_t src_head_stride, int32_t* status) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int64_t slot = batch_id[b];
    const int64_t pos = offset[b];
    if (slot < 0 || slot >= max_batch || pos < 0 || pos >= max_len) {
        if (threadIdx.x == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const T* s = src + b * src_row_stride + h * src_head_stride;
    T* d = cache + ((slot * Hkv + h) * max_len + pos) * kHeadDim;
    for (int i = threadIdx.x; i < kHeadDim; i += blockDim.x) d[i] = s[i];
}

// Scaled logits of one 128-position block of one (row, kv head) for every query head of the group.
// Half a warp per position: lane j of the half owns elements 8j..8j+7 of the key row.
template <typename T>
__global__ void __launch_bounds__(kChainThreads)
qk_kernel(const T* __restrict__ q, const T* __restrict__ key_cache, const int64_t* __restrict__ batch_idx,
          const int32_t* __restrict__ offset, float* __restrict__ logits, int Hq, int Hkv, int64_t max_batch,
          int64_t max_len, int block_seq, float scale, int32_t* status) {
    __shared__ float qs[8][kHeadDim];
    const int b = blockIdx.x, h = blockIdx.y, blk = blockIdx.z;
    const int G = Hq / Hkv;
    const int64_t len = offset[b];
    if ((int64_t)blk * block_seq >= len) return;                       // the reference skips such blocks too
    const int64_t slot = batch_idx[b];
    if (slot < 0 || slot >= max_batch) {
        if (threadIdx.x == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    for (int i = threadIdx.x; i < G * kHeadDim; i += blockDim.x)
        qs[i / kHeadDim][i % kHeadDim] = to_f32(q[((int64_t)b * Hq + (int64_t)h * G) * kHeadDim + i]);
    __syncthreads();
    const int half = threadIdx.x >> 4, j = threadIdx.x & 15;           // 16 half-warps per CTA
    const T* kbase = key_cache + (slot * Hkv + h) * max_len * kHeadDim;
    for (int p = half; p < block_seq; p += kChainThreads / 16) {       // the same trip count for every half-warp
        const int64_t s = (int64_t)blk * block_seq + p;
        const bool valid = s < len && s < max_len;
        float x[8];
        if (valid) load8(kbase + s * kHeadDim + 8 * j, x);
        for (int g = 0; g < G; ++g) {
            float acc = 0.0f;
            if (valid) {
#pragma unroll
                for (int e = 0; e < 8; ++e) acc = fmaf(x[e], qs[g][8 * j + e], acc);
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o, 16);
            if (j == 0 && s < max_len)
                logits[((int64_t)b * Hq + (int64_t)h * G + g) * max_len + s] = valid ? acc * scale : -INFINITY;
        }
    }
}

// blockwise_topk_sparsity on one (row, kv head): keep the sink, the `topk_block` best 16-token blocks
// of the region behind it (block score = mean over the group and the block's 16 logits), and the tail;
// everything else in the region becomes -inf.  Ties go to the lower block.
__global__ void __launch_bounds__(kChainThreads)
block_topk_mask_kernel(float* __restrict__ logits, const int32_t* __restrict__ offset, int Hq, int Hkv,
                       int64_t max_len, int topk_block, int local, int sink, int32_t* status) {
    extern __shared__ float block_score[];           // one per block of the region
    const int b = blockIdx.x, h = blockIdx.y;
    const int G = Hq / Hkv;
    const int64_t len = offset[b];
    int64_t n_full = (int64_t)sink + local + (int64_t)topk_block * kPageSize;
    n_full = (n_full + kPageSize - 1) / kPageSize * kPageSize;
    if (len <= n_full || len > max_len) {
        if (len > max_len && threadIdx.x == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int nblk = (int)((len - local - sink) / kPageSize);
    float* base = logits + ((int64_t)b * Hq + (int64_t)h * G) * max_len + sink;
    for (int n = threadIdx.x; n < nblk; n += blockDim.x) {
        float tot = 0.0f;
        for (int t = 0; t < kPageSize; ++t) {
            float m = 0.0f;
            for (int g = 0; g < G; ++g) m += base[(int64_t)g * max_len + n * kPageSize + t];
            tot += m / (float)G;
        }
        block_score[n] = tot / (float)kPageSize;
    }
    __syncthreads();
    // rank of every block = blocks that beat it (larger score, or equal score and lower index)
    for (int n = threadIdx.x; n < nblk; n += blockDim.x) {
        const float mine = block_score[n];
        int rank = 0;
        for (int m = 0; m < nblk; ++m) {
            const float o = block_score[m];
            rank += (o > mine || (o == mine && m < n)) ? 1 : 0;
        }
        if (rank >= topk_block) {
            for (int g = 0; g < G; ++g)
                for (int t = 0; t < kPageSize; ++t) base[(int64_t)g * max_len + n * kPageSize + t] = -INFINITY;
        }
    }
}

// In-place softmax of logits[row, head, 0 .. offset[row])
__global__ void __launch_bounds__(kChainThreads)
softmax_rows_kernel(float* __restrict__ logits, const int32_t* __restrict__ offset, int Hq, int64_t max_len) {
    __shared__ float red[kChainThreads / 32];
    __shared__ float bcast;
    const int b = blockIdx.x, hq = blockIdx.y;
    int64_t len = offset[b];
    if (len > max_len) len = max_len;
    if (len <= 0) return;
    float* row = logits + ((int64_t)b * Hq + hq) * max_len;
    float mx = -INFINITY;
    for (int64_t s = threadIdx.x; s < len; s += blockDim.x) mx = fmaxf(mx, row[s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = red[0];
        for (int i = 1; i < kChainThreads / 32; ++i) m = fmaxf(m, red[i]);
        bcast = m;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.0f;
    for (int64_t s = threadIdx.x; s < len; s += blockDim.x) {
        const float e = expf(row[s] - mx);
        row[s] = e;
        sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();                       // `red` and `bcast` were read above
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < kChainThreads / 32; ++i) t += red[i];
        bcast = t;
    }
    __syncthreads();
    const float inv = 1.0f / bcast;
    for (int64_t s = threadIdx.x; s < len; s += blockDim.x) row[s] *= inv;
}

// out[row, h*G+g, :] = sum_s p[row, h*G+g, s] * V[batch_idx[row], h, s, :], s < offset[row].
// One CTA per (row, kv head): sixteen half-warps stride over the positions, lane j of a half-warp owns
// elements 8j..8j+7 of the value row; the sixteen partial sums meet in shared memory, in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kChainThreads)
sv_kernel(const T* __restrict__ value_cache, const int64_t* __restrict__ batch_idx,
          const int32_t* __restrict__ offset, const float* __restrict__ probs, T* __restrict__ out, int Hq, int Hkv,
          int64_t max_batch, int64_t max_len, int32_t* status) {
    constexpr int kHalves = kChainThreads / 16;
    __shared__ float red[kHalves][kHeadDim];
    const int b = blockIdx.x, h = blockIdx.y;
    const int G = Hq / Hkv;
    int64_t len = offset[b];
    if (len > max_len) len = max_len;
    const int64_t slot = batch_idx[b];
    if (slot < 0 || slot >= max_batch) {
        if (threadIdx.x == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int half = threadIdx.x >> 4, j = threadIdx.x & 15;
    const T* vbase = value_cache + (slot * Hkv + h) * max_len * kHeadDim;
    const float* pbase = probs + ((int64_t)b * Hq + (int64_t)h * G) * max_len;
    float acc[8][8];
#pragma unroll
    for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
    for (int64_t s = half; s < len; s += kHalves) {
        float x[8];
        load8(vbase + s * kHeadDim + 8 * j, x);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            if (g < G) {
                const float p = pbase[(int64_t)g * max_len + s];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(p, x[e], acc[g][e]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if (g >= G) break;
        __syncthreads();                                   // `red` of the previous head has been read
#pragma unroll
        for (int e = 0; e < 8; ++e) red[half][8 * j + e] = acc[g][e];
        __syncthreads();
        if (threadIdx.x < kHeadDim) {
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < kHalves; ++w) tot += red[w][threadIdx.x];
            out[((int64_t)b * Hq + (int64_t)h * G + g) * kHeadDim + threadIdx.x] = from_f32<T>(tot);
        }
    }
}

}  // namespace ktk

using namespace ktk;

namespace {

int chain_args(const char* who, int32_t rows, int32_t hq, int32_t hkv, int64_t max_batch, int64_t max_len,
               int32_t head_dim, int32_t dtype) {
    if (rows < 0 || hkv <= 0 || hq <= 0 || hq % hkv != 0 || max_batch <= 0 || max_len <= 0) {
        set_error("%s: bad sizes rows=%d heads=%d/%d max_batch=%lld max_len=%lld", who, rows, hq, hkv,
                  (long long)max_batch, (long long)max_len);
        return KTK_ERR_ARG;
    }
    if (dtype != KTK_F32 && dtype != KTK_BF16) {
        set_error("%s: dtype %d is neither KTK_F32 nor KTK_BF16", who, dtype);
        return KTK_ERR_ARG;
    }
    const int g = hq / hkv;
    if (head_dim != kHeadDim || g > 8 || hkv > 65535) {
        set_error("%s: only head_dim=%d, group size <= 8 and <= 65535 kv heads are built", who, kHeadDim);
        return KTK_ERR_UNSUPPORTED;
    }
    return KTK_OK;
}

}  // namespace

extern "C" int ktk_copy_to_cache(void* cache, const void* src, const int64_t* batch_id, const int32_t* offset,
                                 int32_t rows, int32_t num_kv_heads, int64_t max_batch, int64_t max_len,
                                 int32_t head_dim, int64_t src_row_stride, int64_t src_head_stride, int32_t dtype,
                                 int32_t* status, void* stream) {
    int rc = chain_args("ktk_copy_to_cache", rows, num_kv_heads, num_kv_heads, max_batch, max_len, head_dim, dtype);
    if (rc != KTK_OK) return rc;
    if (rows == 0) return KTK_OK;
    if (!cache || !src || !batch_id || !offset) { set_error("ktk_copy_to_cache: null pointer argument"); return KTK_ERR_ARG; }
    const dim3 grid((unsigned)rows, (unsigned)num_kv_heads);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == KTK_F32)
        copy_to_cache_kernel<float><<<grid, 128, 0, st>>>((float*)cache, (const float*)src, batch_id, offset,
                                                         num_kv_heads, max_batch, max_len, src_row_stride,
                                                         src_head_stride, status);
    else
        copy_to_cache_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((__nv_bfloat16*)cache, (const __nv_bfloat16*)src,
                                                                 batch_id, offset, num_kv_heads, max_batch, max_len,
                                                                 src_row_stride, src_head_stride, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_copy_to_cache");
    return KTK_OK;
}

extern "C" int ktk_qk(const void* q, const void* key_cache, const int64_t* batch_idx, const int32_t* offset,
                      float* logits, int32_t rows, int32_t num_q_heads, int32_t num_kv_heads, int64_t max_batch,
                      int64_t max_len, int32_t head_dim, int32_t block_seq, int32_t dtype, int32_t* status,
                      void* stream) {
    int rc = chain_args("ktk_qk", rows, num_q_heads, num_kv_heads, max_batch, max_len, head_dim, dtype);
    if (rc != KTK_OK) return rc;
    if (rows == 0) return KTK_OK;
    if (!q || !key_cache || !batch_idx || !offset || !logits || block_seq <= 0) {
        set_error("ktk_qk: null pointer argument or block_seq <= 0");
        return KTK_ERR_ARG;
    }
    const int64_t blocks = (max_len + block_seq - 1) / block_seq;
    if (blocks > 65535) { set_error("ktk_qk: more than 65535 blocks of %d positions", block_seq); return KTK_ERR_TOO_LARGE; }
    const dim3 grid((unsigned)rows, (unsigned)num_kv_heads, (unsigned)blocks);
    const float scale = 1.0f / sqrtf((float)head_dim);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == KTK_F32)
        qk_kernel<float><<<grid, kChainThreads, 0, st>>>((const float*)q, (const float*)key_cache, batch_idx, offset,
                                                        logits, num_q_heads, num_kv_heads, max_batch, max_len,
                                                        block_seq, scale, status);
    else
        qk_kernel<__nv_bfloat16><<<grid, kChainThreads, 0, st>>>((const __nv_bfloat16*)q,
                                                                (const __nv_bfloat16*)key_cache, batch_idx, offset,
                                                                logits, num_q_heads, num_kv_heads, max_batch,
                                                                max_len, block_seq, scale, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_qk");
    return KTK_OK;
}

extern "C" int ktk_block_topk_mask(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                                   int32_t num_kv_heads, int64_t max_len, int32_t topk_block, int32_t local,
                                   int32_t sink, int32_t* status, void* stream) {
    int rc = chain_args("ktk_block_topk_mask", rows, num_q_heads, num_kv_heads, 1, max_len, kHeadDim, KTK_F32);
    if (rc != KTK_OK) return rc;
    if (rows == 0) return KTK_OK;
    if (!logits || !offset || topk_block < 1 || local < 0 || sink < 0) {
        set_error("ktk_block_topk_mask: null pointer, topk_block < 1, or negative local / sink");
        return KTK_ERR_ARG;
    }
    const size_t smem = (size_t)(max_len / kPageSize + 1) * sizeof(float);
    if (smem > 200 * 1024) { set_error("ktk_block_topk_mask: max_len %lld too long", (long long)max_len); return KTK_ERR_TOO_LARGE; }
    KTK_CUDA_TRY(cudaFuncSetAttribute(block_topk_mask_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                 "ktk_block_topk_mask");
    const dim3 grid((unsigned)rows, (unsigned)num_kv_heads);
    block_topk_mask_kernel<<<grid, kChainThreads, smem, (cudaStream_t)stream>>>(logits, offset, num_q_heads, num_kv_heads,
                                                                               max_len, topk_block, local, sink, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_block_topk_mask");
    return KTK_OK;
}

extern "C" int ktk_softmax_rows(float* logits, const int32_t* offset, int32_t rows, int32_t num_q_heads,
                                int64_t max_len, void* stream) {
    if (rows < 0 || num_q_heads <= 0 || num_q_heads > 65535 || max_len <= 0) {
        set_error("ktk_softmax_rows: bad sizes rows=%d heads=%d max_len=%lld", rows, num_q_heads, (long long)max_len);
        return KTK_ERR_ARG;
    }
    if (rows == 0) return KTK_OK;
    if (!logits || !offset) { set_error("ktk_softmax_rows: null pointer argument"); return KTK_ERR_ARG; }
    const dim3 grid((unsigned)rows, (unsigned)num_q_heads);
    softmax_rows_kernel<<<grid, kChainThreads, 0, (cudaStream_t)stream>>>(logits, offset, num_q_heads, max_len);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_softmax_rows");
    return KTK_OK;
}

extern "C" int ktk_sv(const void* value_cache, const int64_t* batch_idx, const int32_t* offset, const float* probs,
                      void* out, int32_t rows, int32_t num_q_heads, int32_t num_kv_heads, int64_t max_batch,
                      int64_t max_len, int32_t head_dim, int32_t dtype, int32_t* status, void* stream) {
    int rc = chain_args("ktk_sv", rows, num_q_heads, num_kv_heads, max_batch, max_len, head_dim, dtype);
    if (rc != KTK_OK) return rc;
    if (rows == 0) return KTK_OK;
    if (!value_cache || !batch_idx || !offset || !probs || !out) { set_error("ktk_sv: null pointer argument"); return KTK_ERR_ARG; }
    const dim3 grid((unsigned)rows, (unsigned)num_kv_heads);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == KTK_F32)
        sv_kernel<float><<<grid, kChainThreads, 0, st>>>((const float*)value_cache, batch_idx, offset, probs, (float*)out,
                                                        num_q_heads, num_kv_heads, max_batch, max_len, status);
    else
        sv_kernel<__nv_bfloat16><<<grid, kChainThreads, 0, st>>>((const __nv_bfloat16*)value_cache, batch_idx, offset,
                                                                probs, (__nv_bfloat16*)out, num_q_heads, num_kv_heads,
                                                                max_batch, max_len, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_sv");
    return KTK_OK;
}
