// Instantiations of the tcgen05 backward kernel: MODE_DKV, head_dim 64, both half precision
// element types, every (causal, ALiBi, RoPE) composition.
#include "bwd_tcgen05.cuh"

namespace af {
namespace tcb {
AF_DEFINE_BWD_UNIT(launch_dkv_d64, 64, MODE_DKV)
}  // namespace tcb
}  // namespace af
