"""DSL surface: combinators, the @attention decorator and the tracer."""
from .api import (
    attention, scaled_dot_product, additive_bias, rope, causal, sliding_window, full,
    block_sparse, alibi, softmax, relu_attention,
)

__all__ = ["attention", "scaled_dot_product", "additive_bias", "rope", "causal",
           "sliding_window", "full", "block_sparse", "alibi", "softmax", "relu_attention"]
