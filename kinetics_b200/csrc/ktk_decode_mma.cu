// Tensor-core variant of the paged flash-decode (bf16).  Placeholder until the
// TMA-staged kernel lands: reports "not built" so callers fail loudly.
#include "ktk_decode.cuh"

namespace ktk {
int launch_decode_mma(const DecodeParams&, int, cudaStream_t) {
    set_error("ktk decode: the tensor-core variant is not built");
    return KTK_ERR_UNSUPPORTED;
}
}  // namespace ktk
