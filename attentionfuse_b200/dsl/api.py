"""The user-facing DSL: combinators and the ``@attention`` decorator.

Same surface and routing as the reference (attnfuse/dsl/api.py:36-201): combinators build
IR nodes; the decorated function traces once per (head_dim, dtype), then routes a call to
the block-sparse path, the autograd path (when an input requires grad and the graph has a
backward), or the inference launch.  Below this file everything is hand-written sm_100a
CUDA reached through the C-ABI library; there is no CPU fallback.
"""
from __future__ import annotations

import functools
import os
from typing import Callable, Optional

import torch

from ..ir.high_level import (
    Expr, TensorSym, ScoreOp, MaskOp, BiasOp, NormOp, Graph,
    ScoreKind, MaskKind, BiasKind, NormKind,
)
from .tracer import trace_attention_fn


def scaled_dot_product(Q: TensorSym, K: TensorSym, scale: Optional[float] = None) -> Expr:
    """S = (Q @ K^T) * scale; scale defaults to 1/sqrt(head_dim)."""
    return ScoreOp(kind=ScoreKind.SCALED_DOT, q=Q, k=K, scale=scale)


def rope(Q: TensorSym, K: TensorSym, scale: Optional[float] = None) -> Expr:
    """S = (RoPE(Q) @ RoPE(K)^T) * scale with the rotation done inside the kernel.
    Pass the tables at call time: ``fn(Q, K, V, cos=cos, sin=sin)``; shape (N, D) or
    (1, 1, N, D), same dtype as Q (rotate-half convention)."""
    return ScoreOp(kind=ScoreKind.SCALED_DOT, q=Q, k=K, scale=scale, rope=True)


def additive_bias(scores: Expr) -> Expr:
    """S' = S + bias, the (B, H, N, N) tensor given at call time as ``bias=``."""
    return BiasOp(kind=BiasKind.ADDITIVE, scores=scores, bias=None)


def causal(scores: Expr) -> Expr:
    """Mask keys j > i."""
    return MaskOp(kind=MaskKind.CAUSAL, scores=scores)


def sliding_window(scores: Expr, window_size: int) -> Expr:
    """Mask keys with |i - j| >= window_size."""
    if window_size <= 0:
        raise ValueError("sliding_window: window_size must be positive")
    return MaskOp(kind=MaskKind.SLIDING_WINDOW, scores=scores, window=window_size)


def full(scores: Expr) -> Expr:
    """No-op mask."""
    return MaskOp(kind=MaskKind.FULL, scores=scores)


def block_sparse(scores: Expr) -> Expr:
    """Block mask supplied at call time as ``block_mask=<BlockMask>``; only the listed
    (query block, key block) tiles are visited."""
    return MaskOp(kind=MaskKind.BLOCK_SPARSE, scores=scores)


def alibi(scores: Expr, num_heads: int) -> Expr:
    """ALiBi bias  -slope[h] * |i - j|  (Press et al., 2021)."""
    if num_heads <= 0:
        raise ValueError("alibi: num_heads must be positive")
    return BiasOp(kind=BiasKind.ALIBI, scores=scores, num_heads=num_heads)


def softmax(scores: Expr) -> Expr:
    """Row softmax (computed online, tile by tile)."""
    return NormOp(kind=NormKind.SOFTMAX, scores=scores)


def relu_attention(scores: Expr) -> Expr:
    """max(S, 0) normalised by its row sum, in place of softmax."""
    return NormOp(kind=NormKind.RELU, scores=scores)


def _wants_grad(*tensors) -> bool:
    return any(isinstance(t, torch.Tensor) and t.requires_grad for t in tensors)


def attention(fn: Callable) -> Callable:
    """Decorator turning a combinator function into a callable on real Q/K/V tensors."""
    traced: dict = {}

    @functools.wraps(fn)
    def wrapper(Q, K, V, *, bias=None, cos=None, sin=None, block_mask=None,
                return_graph: bool = False, **kwargs):
        key = (Q.shape[-1], Q.dtype)
        entry = traced.get(key)
        if entry is None:
            graph = trace_attention_fn(fn, Q, K, V)
            if os.environ.get("ATTNFUSE_DEBUG"):
                from ..ir.printer import format_graph
                print(f"[AttnFuse] high-level IR (head_dim={key[0]} dtype={key[1]}):")
                print(format_graph(graph))
            # what the routing below needs, looked up once per traced graph instead of per call
            entry = traced[key] = (graph, MaskKind.BLOCK_SPARSE in {m.kind for m in graph.collect_masks()},
                                   any(b.kind is BiasKind.ALIBI for b in graph.collect_biases()), [None])
        graph, is_block_sparse, uses_alibi, backward_ok = entry
        if return_graph:
            return graph

        if is_block_sparse:
            if block_mask is None:
                raise RuntimeError(
                    "a block-sparse graph needs its block lists at call time: "
                    "fn(Q, K, V, block_mask=create_block_mask(predicate, Q_LEN, KV_LEN))")
            from ..runtime.block_mask import BlockMask, run_block_sparse
            if not isinstance(block_mask, BlockMask):
                raise TypeError("block_mask must be an attnfuse.BlockMask")
            bias_kind = 1 if uses_alibi else 0
            if _wants_grad(Q, K, V):
                from ..runtime.autograd import AttnFuseBlockSparseFunction
                return AttnFuseBlockSparseFunction.apply(Q, K, V, block_mask, bias_kind)
            return run_block_sparse(Q, K, V, block_mask, 1.0 / (Q.shape[-1] ** 0.5),
                                    bias_kind=bias_kind)

        if Q.requires_grad or K.requires_grad or V.requires_grad:
            if backward_ok[0] is None:
                from ..runtime.backward import can_backward
                backward_ok[0] = can_backward(graph)
            # a query position offset (chunked prefill against a cache) is forward only
            off = kwargs.get("q_offset")
            if backward_ok[0] and (off is None or (isinstance(off, int) and off == 0)):
                from ..runtime.autograd import AttnFuseFunction
                return AttnFuseFunction.apply(graph, Q, K, V, bias, cos, sin)
            # No backward for this composition: run inference, no gradient flows.

        from ..runtime.dispatch import run_attention
        return run_attention(graph, Q, K, V, bias=bias, cos=cos, sin=sin, **kwargs)

    wrapper.graph_fn = fn
    return wrapper
