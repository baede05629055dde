"""Run the user's attention function once on symbolic tensors to recover its graph.

Reference: attnfuse/dsl/tracer.py:25-85 (4-D (B,H,N,D) inputs only, matching head_dim, and
a ``probs @ V`` root whose probs come from a normalisation combinator).  No device work.
"""
from __future__ import annotations

from typing import Callable

from ..ir.high_level import TensorSym, Graph, MatMulPV, NormOp


def _symbol(name: str, like) -> TensorSym:
    shape = tuple(like.shape)
    if len(shape) != 4:
        raise ValueError(f"AttnFuse expects Q/K/V of shape (B, H, N, D); got {shape}")
    b, h, n, d = shape
    return TensorSym(name=name, batch=b, num_heads=h, seqlen=n, head_dim=d,
                     dtype=str(like.dtype).replace("torch.", ""))


def trace_attention_fn(fn: Callable, Q, K, V) -> Graph:
    q, k, v = _symbol("Q", Q), _symbol("K", K), _symbol("V", V)
    if q.head_dim != k.head_dim:
        raise ValueError(f"head_dim mismatch: Q.head_dim={q.head_dim} K.head_dim={k.head_dim}")
    if v.head_dim != q.head_dim:
        raise ValueError("AttnFuse currently requires Q.head_dim == V.head_dim")
    result = fn(q, k, v)
    if not isinstance(result, MatMulPV):
        raise TypeError(
            f"Attention function must return `probs @ V`; got {type(result).__name__}.  "
            "Did you forget the value projection?")
    if not isinstance(result.probs, NormOp):
        raise TypeError(
            "The attention probabilities passed to `@ V` must come from a "
            "normalisation combinator (af.softmax / af.relu_attention).")
    return Graph(q=q, k=k, v=v, root=result)
