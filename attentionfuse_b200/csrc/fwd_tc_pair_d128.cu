// Instantiations of the two-heads-per-CTA forward kernel: head_dim 128, both half precision
// element types, every (element mask, ALiBi) composition.
#include "fwd_pair_tcgen05.cuh"

namespace af {
namespace tc {
int launch_pair_d128(int dtype, const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                     const CUtensorMap& mo, cudaStream_t st) {
  if (dtype == AF_F16) return launch_pair_composition<__half>(args, mq, mk, mv, mo, st);
  return launch_pair_composition<__nv_bfloat16>(args, mq, mk, mv, mo, st);
}
}  // namespace tc
}  // namespace af
