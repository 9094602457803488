// Host-side plumbing shared by the C entry points: error text, argument checks.
#include <stdarg.h>
#include <stdio.h>

#include "ktk_common.cuh"

namespace ktk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* who) {
    set_error("%s: CUDA error %d (%s)", who, (int)e, cudaGetErrorString(e));
    return KTK_ERR_CUDA;
}

int check_shape(const ktk_shape* s, const char* who) {
    if (s == nullptr) { set_error("%s: shape is null", who); return KTK_ERR_ARG; }
    if (s->batch < 0 || s->num_kv_heads <= 0 || s->group_size <= 0 || s->num_pages < 0) {
        set_error("%s: bad sizes batch=%d num_kv_heads=%d group_size=%d num_pages=%lld", who,
                  s->batch, s->num_kv_heads, s->group_size, (long long)s->num_pages);
        return KTK_ERR_ARG;
    }
    if (s->dtype != KTK_F32 && s->dtype != KTK_BF16) {
        set_error("%s: dtype %d is neither KTK_F32 nor KTK_BF16", who, s->dtype);
        return KTK_ERR_ARG;
    }
    if (s->head_dim != kHeadDim || s->page_size != kPageSize) {
        set_error("%s: only head_dim=%d, page_size=%d are built (got %d, %d)", who, kHeadDim,
                  kPageSize, s->head_dim, s->page_size);
        return KTK_ERR_UNSUPPORTED;
    }
    if (s->group_size != 1 && s->group_size != 2 && s->group_size != 4 && s->group_size != 8) {
        set_error("%s: group_size %d not built (1, 2, 4, 8)", who, s->group_size);
        return KTK_ERR_UNSUPPORTED;
    }
    return KTK_OK;
}

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace ktk

extern "C" const char* ktk_last_error(void) { return ktk::g_err; }
extern "C" const char* ktk_version(void) { return "0.1"; }
