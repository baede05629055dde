// Instantiations of the tcgen05 forward kernel: head_dim 128, RoPE mode ROPE_FUSED, both half
// precision element types, every (element mask, ALiBi) composition.
#include "fwd_tcgen05.cuh"

namespace af {
namespace tc {
AF_DEFINE_TC_UNIT(launch_d128_fused, 128, ROPE_FUSED)
}  // namespace tc
}  // namespace af
