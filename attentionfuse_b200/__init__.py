"""attentionfuse_b200: AttnFuse's attention DSL on hand-written sm_100a CUDA kernels.

Public surface (the reference's, attnfuse/__init__.py:26-58)::

    import attentionfuse_b200 as af

    @af.attention
    def gpt2_attn(Q, K, V):
        s = af.scaled_dot_product(Q, K)
        s = af.causal(s)
        return af.softmax(s) @ V

    out = gpt2_attn(q, k, v)

Underneath, the combinator graph is lowered to the key of a compile-time specialised CUDA
kernel in ``csrc/libattnfuse_b200.so`` (TMA + tcgen05 + TMEM forward, split-K decode,
FA2-style backward, block-sparse variants) and launched through a C ABI.  There is no
Triton, no multi-backend dispatch and no CPU fallback.
"""
from .dsl.api import (
    attention, scaled_dot_product, additive_bias, rope, causal, sliding_window, full,
    block_sparse, alibi, softmax, relu_attention,
)
from .runtime.block_mask import BlockMask, create_block_mask, create_block_mask_per_head

__version__ = "1.0.0"

__all__ = [
    "attention", "scaled_dot_product", "additive_bias", "rope", "causal", "sliding_window",
    "full", "block_sparse", "alibi", "softmax", "relu_attention",
    "BlockMask", "create_block_mask", "create_block_mask_per_head", "__version__",
]
