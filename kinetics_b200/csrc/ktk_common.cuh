// Shared device/host helpers for the block top-k paged decode kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ktk.h"

namespace ktk {

constexpr int kHeadDim = 128;   // D: the only head size built
constexpr int kPageSize = 16;   // P: tokens per page
constexpr int kMaxScoredPages = 32768;  // selection keeps one 32-bit key per page in shared memory

// ---- error plumbing -------------------------------------------------------
void set_error(const char* fmt, ...);
int check_shape(const ktk_shape* s, const char* who);
int cuda_fail(cudaError_t e, const char* who);
int sm_count();
int check_view(const ktk_view* v, const char* who);

// a ktk_view with the defaults filled in
struct View {
    int sink_tokens = 0;
    int local_tokens = 1;
    const int32_t* page_count = nullptr;
    const int32_t* slot_index = nullptr;
    const int32_t* seq_order = nullptr;
};
inline View make_view(const ktk_view* v) {
    View r;
    if (v != nullptr) {
        r.sink_tokens = v->sink_tokens;
        r.local_tokens = v->local_tokens;
        r.page_count = v->page_count;
        r.slot_index = v->slot_index;
        r.seq_order = v->seq_order;
    }
    return r;
}
// most always-attended pages behind the scored ones: 1 + ceil((L - 1) / 16), and 1 for L = 0
inline int view_back_max(int local_tokens) {
    return local_tokens <= 1 ? 1 : 1 + (local_tokens - 1 + kPageSize - 1) / kPageSize;
}
inline int view_row_width(int topk, const View& v) {
    return (v.sink_tokens > 0 ? 1 : 0) + topk + view_back_max(v.local_tokens);
}

#define KTK_CUDA_TRY(expr, who)                        \
    do {                                               \
        cudaError_t _e = (expr);                       \
        if (_e != cudaSuccess) return cuda_fail(_e, who); \
    } while (0)

// ---- element access -------------------------------------------------------
__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// Eight consecutive elements starting at p (16-byte aligned for bf16, 32 for fp32) as fp32.
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void unpack8(const uint4& r, float (&out)[8]) {
    // a bf16 is the upper half of an fp32: widen by shifting
    out[0] = __uint_as_float(r.x << 16); out[1] = __uint_as_float(r.x & 0xffff0000u);
    out[2] = __uint_as_float(r.y << 16); out[3] = __uint_as_float(r.y & 0xffff0000u);
    out[4] = __uint_as_float(r.z << 16); out[5] = __uint_as_float(r.z & 0xffff0000u);
    out[6] = __uint_as_float(r.w << 16); out[7] = __uint_as_float(r.w & 0xffff0000u);
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    unpack8(r, out);
}

// Four consecutive elements as fp32.
__device__ __forceinline__ void load4(const float* p, float (&out)[4]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&out)[4]) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
    out[0] = __uint_as_float(r.x << 16); out[1] = __uint_as_float(r.x & 0xffff0000u);
    out[2] = __uint_as_float(r.y << 16); out[3] = __uint_as_float(r.y & 0xffff0000u);
}

// ---- selection key --------------------------------------------------------
// Order-preserving map fp32 -> uint32 (larger score <=> larger key).  Adding
// +0.0f first folds -0.0 onto +0.0 so that equal scores have equal keys.
__host__ __device__ __forceinline__ uint32_t score_to_key(float s) {
    s = s + 0.0f;
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(s);
#else
    union { float f; uint32_t u; } c; c.f = s; uint32_t u = c.u;
#endif
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// First fault wins; the caller skips the access it was about to make.
__device__ __forceinline__ void report(int32_t* status, int32_t code) {
    if (status != nullptr) atomicCAS(status, KTK_STATUS_OK, code);
}

}  // namespace ktk
