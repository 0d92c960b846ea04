// tcgen05 GEMM (placeholder until the kernel lands: reports "not supported" so the dispatcher uses the
// general-layout path).
#include "contraction.cuh"

namespace mhlo {
bool gemm_tc_supported(const GemmProblem&) { return false; }
int gemm_tc_launch(const GemmProblem&, cudaStream_t) { return fail(MHLO_CUDA_UNSUPPORTED, "tensor-core GEMM not built"); }
bool attention_tc_supported(int, const AttnShape&, const void*) { return false; }
int attention_tc_launch(int, const void*, const void*, const void*, void*, const AttnShape&, cudaStream_t) {
    return fail(MHLO_CUDA_UNSUPPORTED, "tensor-core attention not built");
}
}  // namespace mhlo
