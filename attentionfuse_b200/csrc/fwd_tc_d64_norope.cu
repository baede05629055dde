// Instantiations of the tcgen05 forward kernel: head_dim 64, RoPE mode ROPE_NONE, both half
// precision element types, every (element mask, ALiBi) composition.
#include "fwd_tcgen05.cuh"

namespace af {
namespace tc {
AF_DEFINE_TC_UNIT(launch_d64_norope, 64, ROPE_NONE)
}  // namespace tc
}  // namespace af
