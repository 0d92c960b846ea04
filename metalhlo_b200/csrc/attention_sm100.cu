// tcgen05 flash attention (to be filled in): reports "not supported" so that mhlo_cuda_attention takes the
// general-layout kernel.
#include "contraction.cuh"

namespace mhlo {
int attention_device_error() { return 0; }
bool attention_tc_supported(int, const AttnShape&, const void*) { return false; }
int attention_tc_launch(int, const void*, const void*, const void*, void*, const AttnShape&, cudaStream_t) {
    return fail(MHLO_CUDA_UNSUPPORTED, "tensor-core attention not built");
}
}  // namespace mhlo
