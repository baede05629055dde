// Instantiations of the tcgen05 backward kernel: MODE_DKV, head_dim 128, both half precision
// element types, every (causal, ALiBi, RoPE) composition.
#include "bwd_tcgen05.cuh"

namespace af {
namespace tcb {
AF_DEFINE_BWD_UNIT(launch_dkv_d128, 128, MODE_DKV)
}  // namespace tcb
}  // namespace af
