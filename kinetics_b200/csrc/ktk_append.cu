// Paged KV append with page-summary maintenance, bulk summary rebuild, and the
// two small elementwise/normalisation kernels that sit either side of the
// attention path (RMSNorm, SwiGLU gate).
#include "ktk_common.cuh"

namespace ktk {

int silu_mul_vectorised(const void* gate, const void* up, void* out, int64_t n, int dtype, cudaStream_t st);
int silu_mul_rows(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t in_stride, int dtype,
                  cudaStream_t st);

// One CTA per (sequence, kv head), one thread per head-dim element.
// Writes the new key/value at (last page, last slot) and rewrites that page's
// summary: fp32 sum over slots 0..c-1 in slot order, divided by c, rounded to T.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
append_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ cache,
              T* __restrict__ summaries, int64_t summary_stride,
              const int32_t* __restrict__ kv_indices, const int32_t* __restrict__ kv_indptr,
              const int32_t* __restrict__ kv_last_page_len, const int32_t* __restrict__ page_count,
              const int32_t* __restrict__ slot_index, int Hkv, int64_t num_pages, int32_t* status) {
    const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int beg = kv_indptr[b];
    const int n_pages = page_count ? page_count[b] : kv_indptr[b + 1] - beg;
    const int end = beg + n_pages;
    const int srow_b = slot_index ? slot_index[b] : b;
    if (n_pages <= 0) return;  // empty slot: nothing to append
    const int last = kv_last_page_len[b];
    if (last < 1 || last > kPageSize || (summaries != nullptr && n_pages > summary_stride)) {
        if (d == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int64_t page = kv_indices[end - 1];
    if (page < 0 || page >= num_pages) {
        if (d == 0) report(status, KTK_STATUS_BAD_PAGE);
        return;
    }
    const int slot = last - 1;
    const int64_t row = (int64_t)Hkv * kHeadDim;                 // one token of all heads
    T* kpage = cache + (page * 2) * kPageSize * row + (int64_t)h * kHeadDim + d;
    T* vpage = kpage + kPageSize * row;
    const int64_t src = ((int64_t)b * Hkv + h) * kHeadDim + d;
    const T kn = k[src];
    kpage[slot * row] = kn;
    vpage[slot * row] = v[src];
    if (summaries != nullptr) {
        float acc = 0.0f;
        for (int t = 0; t < slot; ++t) acc = __fadd_rn(acc, to_f32(kpage[t * row]));
        acc = __fadd_rn(acc, to_f32(kn));
        T* srow = summaries + (((int64_t)srow_b * Hkv + h) * summary_stride + (n_pages - 1)) * kHeadDim;
        srow[d] = from_f32<T>(__fdiv_rn(acc, (float)last));
    }
}

// tokens of a sequence of n_pages pages whose last page holds `last` tokens (a sink page holds sink_tokens)
__device__ __forceinline__ int seq_tokens(int n_pages, int last, int sink_tokens) {
    if (sink_tokens == 0) return (n_pages - 1) * kPageSize + last;
    return n_pages == 1 ? last : sink_tokens + (n_pages - 2) * kPageSize + last;
}
// logical page and slot of token `pos`
__device__ __forceinline__ int token_page(int pos, int sink_tokens) {
    if (sink_tokens == 0) return pos / kPageSize;
    return pos < sink_tokens ? 0 : 1 + (pos - sink_tokens) / kPageSize;
}
__device__ __forceinline__ int token_slot(int pos, int sink_tokens) {
    if (sink_tokens == 0) return pos % kPageSize;
    return pos < sink_tokens ? pos : (pos - sink_tokens) % kPageSize;
}

// Several tokens per sequence (prefill, chunked append): token j of the packed k / v belongs to the
// sequence b with append_indptr[b] <= j < append_indptr[b+1] and is the (j - append_indptr[b])-th of the
// sequence's n_app newest tokens.  grid (tokens, Hkv), one thread per head-dim element.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
append_tokens_kernel(const T* __restrict__ k, const T* __restrict__ v, const int32_t* __restrict__ append_indptr,
                     int B, T* __restrict__ cache, const int32_t* __restrict__ kv_indices,
                     const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_last_page_len,
                     const int32_t* __restrict__ page_count, int sink_tokens, int Hkv, int64_t num_pages,
                     int32_t* status) {
    const int j = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    // the sequence that owns token j: last b with append_indptr[b] <= j
    int lo = 0, hi = B;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (append_indptr[mid] <= j) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int a0 = append_indptr[b], n_app = append_indptr[b + 1] - a0;
    if (j < a0 || j >= a0 + n_app) return;                       // token outside every range
    const int beg = kv_indptr[b];
    const int n_pages = page_count ? page_count[b] : kv_indptr[b + 1] - beg;
    const int last = (n_pages > 0) ? kv_last_page_len[b] : 0;
    if (n_pages <= 0 || last < 1 || last > kPageSize) {
        if (d == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int pos = seq_tokens(n_pages, last, sink_tokens) - n_app + (j - a0);
    if (pos < 0) {
        if (d == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int64_t page = kv_indices[beg + token_page(pos, sink_tokens)];
    if (page < 0 || page >= num_pages) {
        if (d == 0) report(status, KTK_STATUS_BAD_PAGE);
        return;
    }
    const int64_t row = (int64_t)Hkv * kHeadDim;
    T* kp = cache + ((page * 2) * kPageSize + token_slot(pos, sink_tokens)) * row + (int64_t)h * kHeadDim + d;
    const int64_t src = ((int64_t)j * Hkv + h) * kHeadDim + d;
    kp[0] = k[src];
    kp[kPageSize * row] = v[src];
}

// grid (B, Hkv, Z): CTA z rebuilds the summaries of logical pages z, z+Z, ...
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
build_summaries_kernel(const T* __restrict__ cache, T* __restrict__ summaries,
                       int64_t summary_stride, const int32_t* __restrict__ kv_indices,
                       const int32_t* __restrict__ kv_indptr,
                       const int32_t* __restrict__ kv_last_page_len, const int32_t* __restrict__ page_count,
                       const int32_t* __restrict__ slot_index, const int32_t* __restrict__ append_indptr,
                       int sink_tokens, int Hkv, int64_t num_pages, int32_t* status) {
    const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int beg = kv_indptr[b];
    const int n_pages = page_count ? page_count[b] : kv_indptr[b + 1] - beg;
    const int srow_b = slot_index ? slot_index[b] : b;
    if (n_pages <= 0) return;
    const int last = kv_last_page_len[b];
    if (last < 1 || last > kPageSize || n_pages > summary_stride) {
        if (d == 0 && blockIdx.z == 0) report(status, KTK_STATUS_BAD_TABLE);
        return;
    }
    const int64_t row = (int64_t)Hkv * kHeadDim;
    T* sbase = summaries + ((int64_t)srow_b * Hkv + h) * summary_stride * kHeadDim + d;
    // after an append of several tokens only the pages they touched need a new summary
    int first = 0;
    if (append_indptr != nullptr) {
        const int n_app = append_indptr[b + 1] - append_indptr[b];
        if (n_app <= 0) return;
        const int len = seq_tokens(n_pages, last, sink_tokens);
        first = token_page(len - n_app < 0 ? 0 : len - n_app, sink_tokens);
    }
    for (int p = first + blockIdx.z; p < n_pages; p += gridDim.z) {
        const int64_t page = kv_indices[beg + p];
        if (page < 0 || page >= num_pages) {
            if (d == 0) report(status, KTK_STATUS_BAD_PAGE);
            continue;
        }
        // a sink page (logical 0 under a view) holds sink_tokens keys unless it is also the last page
        const int c = (p == n_pages - 1) ? last : ((p == 0 && sink_tokens > 0) ? sink_tokens : kPageSize);
        const T* kpage = cache + (page * 2) * kPageSize * row + (int64_t)h * kHeadDim + d;
        float x[kPageSize];
#pragma unroll
        for (int t = 0; t < kPageSize; ++t) x[t] = (t < c) ? to_f32(kpage[t * row]) : 0.0f;
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < kPageSize; ++t)
            if (t < c) acc = __fadd_rn(acc, x[t]);
        sbase[(int64_t)p * kHeadDim] = from_f32<T>(__fdiv_rn(acc, (float)c));
    }
}

// ---- RMSNorm --------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// cols == 128: one warp per row, four elements per lane.
template <typename T>
__global__ void __launch_bounds__(128)
rmsnorm128_kernel(const T* __restrict__ x, const T* __restrict__ w, float eps,
                  T* __restrict__ out, int64_t rows) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= rows) return;
    float xv[4], wv[4];
    load4(x + r * 128 + lane * 4, xv);
    load4(w + lane * 4, wv);
    float ss = xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
    T* o = out + r * 128 + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = from_f32<T>(xv[i] * inv * wv[i]);
}

// general cols: one 256-thread CTA per row.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w, float eps, T* __restrict__ out,
               int cols) {
    __shared__ float part[8];
    const int64_t r = blockIdx.x;
    const T* xr = x + r * cols;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float f = to_f32(xr[c]);
        ss += f * f;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = rsqrtf(tot / (float)cols + eps);
    T* o = out + r * cols;
    for (int c = threadIdx.x; c < cols; c += 256)
        o[c] = from_f32<T>(to_f32(xr[c]) * inv * to_f32(w[c]));
}

template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float g = to_f32(gate[i]);
        const float s = g / (1.0f + __expf(-g));
        out[i] = from_f32<T>(s * to_f32(up[i]));
    }
}

template <typename T>
static int append_impl(const void* k, const void* v, void* cache, void* summaries,
                       int64_t summary_stride, const int32_t* kv_indices,
                       const int32_t* kv_indptr, const int32_t* kv_last_page_len, const View& view,
                       const ktk_shape* s, int32_t* status, cudaStream_t st) {
    dim3 grid(s->batch, s->num_kv_heads);
    append_kernel<T><<<grid, kHeadDim, 0, st>>>(
        (const T*)k, (const T*)v, (T*)cache, (T*)summaries, summary_stride, kv_indices, kv_indptr,
        kv_last_page_len, view.page_count, view.slot_index, s->num_kv_heads, s->num_pages, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_append");
    return KTK_OK;
}

template <typename T>
static int build_impl(const void* cache, void* summaries, int64_t summary_stride,
                      const int32_t* kv_indices, const int32_t* kv_indptr,
                      const int32_t* kv_last_page_len, const View& view, const ktk_shape* s, int32_t* status,
                      cudaStream_t st, const int32_t* append_indptr = nullptr) {
    const int64_t bh = (int64_t)s->batch * s->num_kv_heads;
    int z = (int)((8LL * sm_count() + bh - 1) / bh);
    if (z < 1) z = 1;
    if (z > 64) z = 64;
    dim3 grid(s->batch, s->num_kv_heads, z);
    build_summaries_kernel<T><<<grid, kHeadDim, 0, st>>>(
        (const T*)cache, (T*)summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
        view.page_count, view.slot_index, append_indptr, view.sink_tokens, s->num_kv_heads, s->num_pages, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_build_summaries");
    return KTK_OK;
}

}  // namespace ktk

using namespace ktk;

extern "C" int ktk_append_v(const void* k, const void* v, void* kv_cache, void* summaries,
                            int64_t summary_stride, const int32_t* kv_indices,
                            const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                            const ktk_view* view_in, const ktk_shape* shape, int32_t* status, void* stream) {
    int rc = check_shape(shape, "ktk_append");
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, "ktk_append");
    if (rc != KTK_OK) return rc;
    if (shape->batch == 0) return KTK_OK;
    if (!k || !v || !kv_cache || !kv_indices || !kv_indptr || !kv_last_page_len) {
        set_error("ktk_append: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (summaries != nullptr && summary_stride <= 0) {
        set_error("ktk_append: summary_stride must be positive (got %lld)", (long long)summary_stride);
        return KTK_ERR_ARG;
    }
    const View view = make_view(view_in);
    cudaStream_t st = (cudaStream_t)stream;
    if (shape->dtype == KTK_F32)
        return append_impl<float>(k, v, kv_cache, summaries, summary_stride, kv_indices, kv_indptr,
                                  kv_last_page_len, view, shape, status, st);
    return append_impl<__nv_bfloat16>(k, v, kv_cache, summaries, summary_stride, kv_indices,
                                      kv_indptr, kv_last_page_len, view, shape, status, st);
}

extern "C" int ktk_append(const void* k, const void* v, void* kv_cache, void* summaries,
                          int64_t summary_stride, const int32_t* kv_indices,
                          const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                          const ktk_shape* shape, int32_t* status, void* stream) {
    return ktk_append_v(k, v, kv_cache, summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
                        nullptr, shape, status, stream);
}

extern "C" int ktk_build_summaries_v(const void* kv_cache, void* summaries, int64_t summary_stride,
                                     const int32_t* kv_indices, const int32_t* kv_indptr,
                                     const int32_t* kv_last_page_len, const ktk_view* view_in,
                                     const ktk_shape* shape, int32_t* status, void* stream) {
    int rc = check_shape(shape, "ktk_build_summaries");
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, "ktk_build_summaries");
    if (rc != KTK_OK) return rc;
    if (shape->batch == 0) return KTK_OK;
    if (!kv_cache || !summaries || !kv_indices || !kv_indptr || !kv_last_page_len) {
        set_error("ktk_build_summaries: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (summary_stride <= 0) {
        set_error("ktk_build_summaries: summary_stride must be positive");
        return KTK_ERR_ARG;
    }
    const View view = make_view(view_in);
    cudaStream_t st = (cudaStream_t)stream;
    if (shape->dtype == KTK_F32)
        return build_impl<float>(kv_cache, summaries, summary_stride, kv_indices, kv_indptr,
                                 kv_last_page_len, view, shape, status, st);
    return build_impl<__nv_bfloat16>(kv_cache, summaries, summary_stride, kv_indices, kv_indptr,
                                     kv_last_page_len, view, shape, status, st);
}

extern "C" int ktk_append_tokens(const void* k, const void* v, const int32_t* append_indptr, int64_t total_tokens,
                                 void* kv_cache, void* summaries, int64_t summary_stride,
                                 const int32_t* kv_indices, const int32_t* kv_indptr,
                                 const int32_t* kv_last_page_len, const ktk_view* view_in, const ktk_shape* shape,
                                 int32_t* status, void* stream) {
    int rc = check_shape(shape, "ktk_append_tokens");
    if (rc != KTK_OK) return rc;
    rc = check_view(view_in, "ktk_append_tokens");
    if (rc != KTK_OK) return rc;
    if (total_tokens < 0 || total_tokens > 2147483647LL) {
        set_error("ktk_append_tokens: total_tokens %lld out of range", (long long)total_tokens);
        return KTK_ERR_ARG;
    }
    if (shape->batch == 0 || total_tokens == 0) return KTK_OK;
    if (!k || !v || !append_indptr || !kv_cache || !kv_indices || !kv_indptr || !kv_last_page_len) {
        set_error("ktk_append_tokens: null pointer argument");
        return KTK_ERR_ARG;
    }
    if (summaries != nullptr && summary_stride <= 0) {
        set_error("ktk_append_tokens: summary_stride must be positive");
        return KTK_ERR_ARG;
    }
    const View view = make_view(view_in);
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)total_tokens, shape->num_kv_heads);
    if (shape->dtype == KTK_F32)
        append_tokens_kernel<float><<<grid, kHeadDim, 0, st>>>(
            (const float*)k, (const float*)v, append_indptr, shape->batch, (float*)kv_cache, kv_indices, kv_indptr,
            kv_last_page_len, view.page_count, view.sink_tokens, shape->num_kv_heads, shape->num_pages, status);
    else
        append_tokens_kernel<__nv_bfloat16><<<grid, kHeadDim, 0, st>>>(
            (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, append_indptr, shape->batch, (__nv_bfloat16*)kv_cache,
            kv_indices, kv_indptr, kv_last_page_len, view.page_count, view.sink_tokens, shape->num_kv_heads,
            shape->num_pages, status);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_append_tokens");
    if (summaries == nullptr) return KTK_OK;
    if (shape->dtype == KTK_F32)
        return build_impl<float>(kv_cache, summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len, view,
                                 shape, status, st, append_indptr);
    return build_impl<__nv_bfloat16>(kv_cache, summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
                                     view, shape, status, st, append_indptr);
}

extern "C" int ktk_build_summaries(const void* kv_cache, void* summaries, int64_t summary_stride,
                                   const int32_t* kv_indices, const int32_t* kv_indptr,
                                   const int32_t* kv_last_page_len, const ktk_shape* shape,
                                   int32_t* status, void* stream) {
    return ktk_build_summaries_v(kv_cache, summaries, summary_stride, kv_indices, kv_indptr, kv_last_page_len,
                                 nullptr, shape, status, stream);
}

extern "C" int ktk_rmsnorm(const void* x, const void* w, float eps, void* out, int64_t rows,
                           int32_t cols, int32_t dtype, void* stream) {
    if (rows < 0 || cols <= 0 || (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_rmsnorm: bad arguments rows=%lld cols=%d dtype=%d", (long long)rows, cols, dtype);
        return KTK_ERR_ARG;
    }
    if (rows == 0) return KTK_OK;
    if (!x || !w || !out) { set_error("ktk_rmsnorm: null pointer argument"); return KTK_ERR_ARG; }
    if (rows > 2147483647LL) { set_error("ktk_rmsnorm: too many rows"); return KTK_ERR_TOO_LARGE; }
    cudaStream_t st = (cudaStream_t)stream;
    if (cols == 128) {
        const unsigned grid = (unsigned)((rows + 3) / 4);
        if (dtype == KTK_F32)
            rmsnorm128_kernel<float><<<grid, 128, 0, st>>>((const float*)x, (const float*)w, eps, (float*)out, rows);
        else
            rmsnorm128_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out, rows);
    } else {
        if (dtype == KTK_F32)
            rmsnorm_kernel<float><<<(unsigned)rows, 256, 0, st>>>((const float*)x, (const float*)w, eps, (float*)out, cols);
        else
            rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(
                (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out, cols);
    }
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_rmsnorm");
    return KTK_OK;
}

extern "C" int ktk_silu_mul_rows(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                                 int64_t in_row_stride, int32_t dtype, void* stream) {
    const int64_t esz = dtype == KTK_F32 ? 4 : 2;
    if (rows < 0 || cols < 0 || in_row_stride < cols || (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_silu_mul_rows: bad arguments rows=%lld cols=%lld stride=%lld dtype=%d", (long long)rows,
                  (long long)cols, (long long)in_row_stride, dtype);
        return KTK_ERR_ARG;
    }
    if (rows == 0 || cols == 0) return KTK_OK;
    if (!gate || !up || !out) { set_error("ktk_silu_mul_rows: null pointer argument"); return KTK_ERR_ARG; }
    if (cols % 8 != 0 || (in_row_stride * esz) % 16 != 0 ||
        ((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) & 15u) != 0)) {
        set_error("ktk_silu_mul_rows: cols must be a multiple of 8 and rows 16-byte aligned");
        return KTK_ERR_ARG;
    }
    return silu_mul_rows(gate, up, out, rows, cols, in_row_stride, dtype, (cudaStream_t)stream);
}

extern "C" int ktk_silu_mul(const void* gate, const void* up, void* out, int64_t n, int32_t dtype,
                            void* stream) {
    if (n < 0 || (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_silu_mul: bad arguments n=%lld dtype=%d", (long long)n, dtype);
        return KTK_ERR_ARG;
    }
    if (n == 0) return KTK_OK;
    if (!gate || !up || !out) { set_error("ktk_silu_mul: null pointer argument"); return KTK_ERR_ARG; }
    cudaStream_t st = (cudaStream_t)stream;
    if (n % 8 == 0 && ((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) & 15u) == 0))
        return silu_mul_vectorised(gate, up, out, n, dtype, st);
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (dtype == KTK_F32)
        silu_mul_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)gate, (const float*)up, (float*)out, n);
    else
        silu_mul_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
            (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)out, n);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_silu_mul");
    return KTK_OK;
}
