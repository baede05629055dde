// Instantiations of the tcgen05 backward kernel: MODE_FUSED (single pass, dQ through an fp32
// accumulator), head_dim 128, both half precision element types, every (mask, ALiBi, RoPE)
// composition.
#include "bwd_tcgen05.cuh"

namespace af {
namespace tcb {
AF_DEFINE_BWD_UNIT(launch_fused_d128, 128, MODE_FUSED)
}  // namespace tcb
}  // namespace af
