// Host-side plumbing shared by the C entry points: error text, argument checks.
#include <stdarg.h>
#include <stdio.h>

#include "ktk_common.cuh"
#include "ktk_pipeline.cuh"

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

int check_view(const ktk_view* v, const char* who) {
    if (v == nullptr) return KTK_OK;
    if (v->sink_tokens < 0 || v->sink_tokens >= kPageSize || v->local_tokens < 0 || v->local_tokens > (1 << 24)) {
        set_error("%s: view with sink_tokens=%d (0..%d), local_tokens=%d (>= 0)", who, v->sink_tokens,
                  kPageSize - 1, v->local_tokens);
        return KTK_ERR_ARG;
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

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that
// the library carries no link-time dependency on libcuda (it must load on machines without a GPU).
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

int make_tensor_map_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, const uint64_t dims[3],
                       const uint64_t strides_bytes[2], const uint32_t box[3], CUtensorMapSwizzle swizzle,
                       const char* who) {
    static encode_tiled_fn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return cuda_fail(e, who);
        if (qres != cudaDriverEntryPointSuccess || fn == nullptr) {
            set_error("%s: the driver does not provide cuTensorMapEncodeTiled", who);
            return KTK_ERR_CUDA;
        }
        encode = (encode_tiled_fn)fn;
    }
    cuuint64_t gdim[3] = {dims[0], dims[1], dims[2]};
    cuuint64_t gstr[2] = {strides_bytes[0], strides_bytes[1]};
    cuuint32_t bx[3] = {box[0], box[1], box[2]};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = encode(out, dt, 3, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("%s: cuTensorMapEncodeTiled failed with %d (base %p, dims %llu x %llu x %llu)", who, (int)r,
                  base, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2]);
        return KTK_ERR_CUDA;
    }
    return KTK_OK;
}

}  // namespace ktk

extern "C" const char* ktk_last_error(void) { return ktk::g_err; }
extern "C" const char* ktk_version(void) { return "0.3"; }
extern "C" int32_t ktk_view_row_width(int32_t topk, const ktk_view* view) {
    if (ktk::check_view(view, "ktk_view_row_width") != KTK_OK || topk < 0) return -1;
    return ktk::view_row_width(topk, ktk::make_view(view));
}
