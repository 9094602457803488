// Cross-rank helpers shared by the NVLink exchange kernels: system-scope flag stores and polls,
// NVSwitch multicast loads (multimem.ld_reduce) and stores (multimem.st).
#pragma once

#include "ktk_common.cuh"

namespace ktk {

constexpr int kCommThreads = 256;
constexpr int kCommMaxVec = 4;          // vectors of 8 elements per thread: cols <= 8192
constexpr int kCommMaxWorld = 16;
constexpr uint32_t kCommSpinCap = 1u << 24;   // ~ a second of polling

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// eight bf16 summed over all ranks by the switch (fp32 accumulation), returned as four bf16x2
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
    uint4 r;
    // no "memory" clobber: the loads of a row may be in flight together; the barrier before them
    // (bar.sync) already keeps them behind the flag waits
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc_addr));
    return r;
}
// sixteen bytes to every rank of the multicast object
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w))
                 : "memory");
}

// Same-index CTAs of all ranks signal one another: flags[p] is rank p's flag array, [CTA][source rank].
// Tell every peer that this CTA reached `value` (all of the CTA's earlier writes come first).
__device__ __forceinline__ void cta_signal_all_ranks(uint32_t* const* flags, int rank, int world, uint32_t value) {
    __syncthreads();
    if ((int)threadIdx.x < world)
        st_release_sys(flags[threadIdx.x] + (size_t)blockIdx.x * world + rank, value);
}
// Wait until the same-index CTA of rank `src` said `value` (bounded).
__device__ __forceinline__ void flag_wait(const uint32_t* mine, uint32_t value, int32_t* status) {
    for (uint32_t i = 0; i < kCommSpinCap; ++i) {
        if ((int32_t)(ld_acquire_sys(mine) - value) >= 0) return;
        if (i > 64) __nanosleep(64);
    }
    report(status, KTK_STATUS_TIMEOUT);
}
__device__ __forceinline__ void cta_wait_rank(uint32_t* const* flags, int rank, int world, int src, uint32_t value,
                                              int32_t* status) {
    if (threadIdx.x == 0) flag_wait(flags[rank] + (size_t)blockIdx.x * world + src, value, status);
    __syncthreads();
}
__device__ __forceinline__ void cta_wait_all_ranks(uint32_t* const* flags, int rank, int world, uint32_t value,
                                                   int32_t* status) {
    if ((int)threadIdx.x < world) flag_wait(flags[rank] + (size_t)blockIdx.x * world + threadIdx.x, value, status);
    __syncthreads();
}

}  // namespace ktk
