// Tensor-core backward (placeholder translation unit until the kernels land): reports that no
// composition is supported so that af_bwd runs the exact FFMA kernels.
#include "common.cuh"

namespace af {

bool bwd_mma_supports(const AfBwdParams&, const char** why) {
  if (why) *why = "no tensor-core backward instantiation";
  return false;
}

int launch_bwd_mma(const AfBwdParams&, cudaStream_t) {
  return fail(AF_ERR_UNSUPPORTED, "no tensor-core backward instantiation");
}

}  // namespace af
