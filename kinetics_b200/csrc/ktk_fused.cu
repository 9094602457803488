// Fused element-wise kernels around the attention path of the decoder layer:
//   residual add + RMSNorm in one pass, and the split of the fused QKV projection
//   into q-norm, k-norm and v in one launch.  All are HBM-bound streams; every
//   thread moves 16 bytes per access.
#include "ktk_common.cuh"

namespace ktk {

// eight consecutive elements
template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        unpack8(*reinterpret_cast<const uint4*>(p), f);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint4 r;
        __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(f[4], f[5]), d = __floats2bfloat162_rn(f[6], f[7]);
        r.x = *reinterpret_cast<uint32_t*>(&a); r.y = *reinterpret_cast<uint32_t*>(&b);
        r.z = *reinterpret_cast<uint32_t*>(&c); r.w = *reinterpret_cast<uint32_t*>(&d);
        *reinterpret_cast<uint4*>(p) = r;
    }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *(reinterpret_cast<float4*>(p) + 1) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

__device__ __forceinline__ float warp_sum_f(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;     // a thread keeps up to 4 x 8 elements of its row: cols <= 8192

// One CTA per row.  s = x (+ residual); out_sum = s (if asked); out_norm = s * rsqrt(mean(s^2) + eps) * w.
// The sum is rounded to T before it is normalised, as it would be if it had been stored and re-read.
template <typename T>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w, float eps,
                   T* __restrict__ out_sum, T* __restrict__ out_norm, int cols) {
    __shared__ float part[kNormThreads / 32];
    const int64_t r = blockIdx.x;
    const int nvec = cols / 8;
    float v[kNormMaxVec][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c < nvec) {
            Vec8<T>::load(x + r * cols + c * 8, v[i]);
            if (residual != nullptr) {
                float t[8];
                Vec8<T>::load(residual + r * cols + c * 8, t);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] = to_f32(from_f32<T>(v[i][e] + t[e]));
                if (out_sum != nullptr) Vec8<T>::store(out_sum + r * cols + c * 8, v[i]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
        }
    }
    ss = warp_sum_f(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) tot += part[i];
    const float inv = rsqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int c = threadIdx.x + i * kNormThreads;
        if (c < nvec) {
            float wv[8], o[8];
            Vec8<T>::load(w + c * 8, wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = v[i][e] * inv * wv[e];
            Vec8<T>::store(out_norm + r * cols + c * 8, o);
        }
    }
}

// One warp per head row of the fused projection [B, (Hq + 2 Hkv) * 128]:
// query heads -> RMSNorm with wq -> q[B, Hq, 128]; key heads -> RMSNorm with wk -> k[B, Hkv, 128];
// value heads -> copied to v[B, Hkv, 128].  With kRope the normalised query and key heads are then
// rotated, x * cos[pos] + rotate_half(x) * sin[pos] with rotate_half(x) = (-x[64:], x[:64]) and
// pos = position_ids[b]; cos / sin are [max_positions, 128] tables in the model dtype.
template <typename T, bool kRope>
__global__ void __launch_bounds__(128)
qkv_norm_kernel(const T* __restrict__ proj, const T* __restrict__ wq, const T* __restrict__ wk, float eps,
                T* __restrict__ q, T* __restrict__ k, T* __restrict__ v, int64_t rows, int Hq, int Hkv,
                const T* __restrict__ cos_tab, const T* __restrict__ sin_tab,
                const int64_t* __restrict__ position_ids, int64_t max_positions) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int heads = Hq + 2 * Hkv;
    const int64_t b = row / heads;
    const int hh = (int)(row % heads);
    float xv[4];
    load4(proj + row * kHeadDim + lane * 4, xv);
    T* dst;
    const T* wsel = nullptr;
    if (hh < Hq) { dst = q + (b * Hq + hh) * kHeadDim; wsel = wq; }
    else if (hh < Hq + Hkv) { dst = k + (b * Hkv + (hh - Hq)) * kHeadDim; wsel = wk; }
    else { dst = v + (b * Hkv + (hh - Hq - Hkv)) * kHeadDim; }
    float ss = xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3];
    ss = warp_sum_f(ss);
    float o[4] = {xv[0], xv[1], xv[2], xv[3]};
    if (wsel != nullptr) {
        float wv[4];
        load4(wsel + lane * 4, wv);
        const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = xv[i] * inv * wv[i];
        if constexpr (kRope) {
            int64_t pos = position_ids[b];
            pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
            float c[4], sn[4];
            load4(cos_tab + pos * kHeadDim + lane * 4, c);
            load4(sin_tab + pos * kHeadDim + lane * 4, sn);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x = to_f32(from_f32<T>(o[i]));            // the norm's output is a tensor of the model dtype
                const float other = __shfl_xor_sync(0xffffffffu, x, 16);   // element i +- 64
                o[i] = x * c[i] + (lane < 16 ? -other : other) * sn[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[lane * 4 + i] = from_f32<T>(o[i]);
}

// out = silu(gate) * up, eight elements per thread and access
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_vec_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += stride) {
        float g[8], u[8], o[8];
        Vec8<T>::load(gate + i * 8, g);
        Vec8<T>::load(up + i * 8, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.0f + __expf(-g[e])) * u[e];
        Vec8<T>::store(out + i * 8, o);
    }
}

// the same over [rows, cols] operands whose rows lie `in_stride` elements apart (the two halves of one GEMM
// output [rows, 2 * cols]); `out` is contiguous
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_rows_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t rows,
                     int64_t vec_per_row, int64_t in_stride) {
    const int64_t nvec = rows * vec_per_row;
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nvec; i += stride) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 8;
        float g[8], u[8], o[8];
        Vec8<T>::load(gate + r * in_stride + c, g);
        Vec8<T>::load(up + r * in_stride + c, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.0f + __expf(-g[e])) * u[e];
        Vec8<T>::store(out + i * 8, o);
    }
}

template <typename T>
static int add_rmsnorm_launch(const void* x, const void* residual, const void* w, float eps, void* out_sum,
                              void* out_norm, int64_t rows, int cols, cudaStream_t st) {
    add_rmsnorm_kernel<T><<<(unsigned)rows, kNormThreads, 0, st>>>((const T*)x, (const T*)residual, (const T*)w,
                                                                   eps, (T*)out_sum, (T*)out_norm, cols);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_add_rmsnorm");
    return KTK_OK;
}

template <typename T>
static int qkv_norm_launch(const void* proj, const void* wq, const void* wk, float eps, void* q, void* k, void* v,
                           int64_t rows, int Hq, int Hkv, const void* cos_tab, const void* sin_tab,
                           const int64_t* position_ids, int64_t max_positions, cudaStream_t st) {
    const unsigned grid = (unsigned)((rows + 3) / 4);
    if (cos_tab != nullptr)
        qkv_norm_kernel<T, true><<<grid, 128, 0, st>>>((const T*)proj, (const T*)wq, (const T*)wk, eps, (T*)q, (T*)k,
                                                       (T*)v, rows, Hq, Hkv, (const T*)cos_tab, (const T*)sin_tab,
                                                       position_ids, max_positions);
    else
        qkv_norm_kernel<T, false><<<grid, 128, 0, st>>>((const T*)proj, (const T*)wq, (const T*)wk, eps, (T*)q, (T*)k,
                                                        (T*)v, rows, Hq, Hkv, nullptr, nullptr, nullptr, 0);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_qkv_norm");
    return KTK_OK;
}

template <typename T>
static int silu_vec_launch(const void* gate, const void* up, void* out, int64_t nvec, cudaStream_t st) {
    int64_t blocks = (nvec + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    silu_mul_vec_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T*)gate, (const T*)up, (T*)out, nvec);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_silu_mul");
    return KTK_OK;
}

template <typename T>
static int silu_rows_launch(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t in_stride,
                            cudaStream_t st) {
    const int64_t nvec = rows * (cols / 8);
    int64_t blocks = (nvec + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    silu_mul_rows_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T*)gate, (const T*)up, (T*)out, rows, cols / 8,
                                                               in_stride);
    KTK_CUDA_TRY(cudaGetLastError(), "ktk_silu_mul_rows");
    return KTK_OK;
}

int silu_mul_rows(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t in_stride, int dtype,
                  cudaStream_t st) {
    return dtype == KTK_F32 ? silu_rows_launch<float>(gate, up, out, rows, cols, in_stride, st)
                            : silu_rows_launch<__nv_bfloat16>(gate, up, out, rows, cols, in_stride, st);
}

// used by ktk_silu_mul when the length and the pointers allow 16-byte accesses
int silu_mul_vectorised(const void* gate, const void* up, void* out, int64_t n, int dtype, cudaStream_t st) {
    return dtype == KTK_F32 ? silu_vec_launch<float>(gate, up, out, n / 8, st)
                            : silu_vec_launch<__nv_bfloat16>(gate, up, out, n / 8, st);
}

}  // namespace ktk

using namespace ktk;

extern "C" int ktk_add_rmsnorm(const void* x, const void* residual, const void* w, float eps, void* out_sum,
                               void* out_norm, int64_t rows, int32_t cols, int32_t dtype, void* stream) {
    if (rows < 0 || cols <= 0 || (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_add_rmsnorm: bad arguments rows=%lld cols=%d dtype=%d", (long long)rows, cols, dtype);
        return KTK_ERR_ARG;
    }
    if (rows == 0) return KTK_OK;
    if (!x || !w || !out_norm) { set_error("ktk_add_rmsnorm: null pointer argument"); return KTK_ERR_ARG; }
    if (cols % 8 != 0 || cols > 8 * kNormThreads * kNormMaxVec) {
        set_error("ktk_add_rmsnorm: cols must be a multiple of 8 and at most %d (got %d)",
                  8 * kNormThreads * kNormMaxVec, cols);
        return KTK_ERR_UNSUPPORTED;
    }
    const uintptr_t al = (uintptr_t)x | (uintptr_t)w | (uintptr_t)out_norm | (uintptr_t)residual | (uintptr_t)out_sum;
    if ((al & 15u) != 0) { set_error("ktk_add_rmsnorm: pointers must be 16-byte aligned"); return KTK_ERR_ARG; }
    if (rows > 2147483647LL) { set_error("ktk_add_rmsnorm: too many rows"); return KTK_ERR_TOO_LARGE; }
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == KTK_F32 ? add_rmsnorm_launch<float>(x, residual, w, eps, out_sum, out_norm, rows, cols, st)
                            : add_rmsnorm_launch<__nv_bfloat16>(x, residual, w, eps, out_sum, out_norm, rows, cols, st);
}

extern "C" int ktk_qkv_norm(const void* proj, const void* wq, const void* wk, float eps, void* q, void* k, void* v,
                            int64_t batch, int32_t num_q_heads, int32_t num_kv_heads, int32_t dtype, void* stream) {
    if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_qkv_norm: bad arguments batch=%lld Hq=%d Hkv=%d dtype=%d", (long long)batch, num_q_heads,
                  num_kv_heads, dtype);
        return KTK_ERR_ARG;
    }
    if (batch == 0) return KTK_OK;
    if (!proj || !wq || !wk || !q || !k || !v) { set_error("ktk_qkv_norm: null pointer argument"); return KTK_ERR_ARG; }
    const int64_t rows = batch * (num_q_heads + 2 * num_kv_heads);
    if ((rows + 3) / 4 > 2147483647LL) { set_error("ktk_qkv_norm: too many rows"); return KTK_ERR_TOO_LARGE; }
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == KTK_F32 ? qkv_norm_launch<float>(proj, wq, wk, eps, q, k, v, rows, num_q_heads, num_kv_heads,
                                                     nullptr, nullptr, nullptr, 0, st)
                            : qkv_norm_launch<__nv_bfloat16>(proj, wq, wk, eps, q, k, v, rows, num_q_heads,
                                                             num_kv_heads, nullptr, nullptr, nullptr, 0, st);
}

extern "C" int ktk_qkv_norm_rope(const void* proj, const void* wq, const void* wk, float eps, const void* cos_table,
                                 const void* sin_table, const int64_t* position_ids, int64_t max_positions, void* q,
                                 void* k, void* v, int64_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t dtype, void* stream) {
    if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_positions <= 0 ||
        (dtype != KTK_F32 && dtype != KTK_BF16)) {
        set_error("ktk_qkv_norm_rope: bad arguments batch=%lld Hq=%d Hkv=%d positions=%lld dtype=%d", (long long)batch,
                  num_q_heads, num_kv_heads, (long long)max_positions, dtype);
        return KTK_ERR_ARG;
    }
    if (batch == 0) return KTK_OK;
    if (!proj || !wq || !wk || !q || !k || !v || !cos_table || !sin_table || !position_ids) {
        set_error("ktk_qkv_norm_rope: null pointer argument");
        return KTK_ERR_ARG;
    }
    const int64_t rows = batch * (num_q_heads + 2 * num_kv_heads);
    if ((rows + 3) / 4 > 2147483647LL) { set_error("ktk_qkv_norm_rope: too many rows"); return KTK_ERR_TOO_LARGE; }
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == KTK_F32
               ? qkv_norm_launch<float>(proj, wq, wk, eps, q, k, v, rows, num_q_heads, num_kv_heads, cos_table,
                                        sin_table, position_ids, max_positions, st)
               : qkv_norm_launch<__nv_bfloat16>(proj, wq, wk, eps, q, k, v, rows, num_q_heads, num_kv_heads, cos_table,
                                                sin_table, position_ids, max_positions, st);
}
