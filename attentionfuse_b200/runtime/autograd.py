"""torch.autograd bindings (reference: attnfuse/runtime/autograd.py:31-97).

Forward saves (Q, K, V, O, L) with L the fp32 log-sum-exp written by the forward kernel;
backward calls the backward launch.  Unlike the reference, the scale saved for backward is
the one the forward used (a custom ``scale=`` is honoured) and RoPE graphs are supported.
"""
from __future__ import annotations

import torch

from .backward import can_backward, run_backward
from .dispatch import run_attention
from .kernel_cache import get_or_compile


class AttnFuseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, graph, Q, K, V, bias, cos, sin):
        if not can_backward(graph):
            raise RuntimeError(
                "AttnFuse backward supports softmax graphs with dense, causal or sliding-window "
                "masks; got a graph outside that scope. Call .detach() on Q/K/V to use the "
                "inference path.")
        B, H_q, N_q, _ = Q.shape
        L = torch.empty(B, H_q, N_q, dtype=torch.float32, device=Q.device)
        kept: list = []
        out = run_attention(graph, Q, K, V, bias=bias, cos=cos, sin=sin, save_lse=L, keep_workspace=kept)
        # RoPE: the forward's workspace holds the rotated Q and K; the backward takes it over
        ctx.rotated = kept[0] if kept else None
        ctx.graph = graph
        ctx.sm_scale = get_or_compile(graph).sm_scale
        ctx.bias, ctx.cos, ctx.sin = bias, cos, sin
        ctx.save_for_backward(Q, K, V, out, L)
        return out

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, O, L = ctx.saved_tensors
        dQ, dK, dV = run_backward(ctx.graph, Q, K, V, O, L, dO.contiguous(), ctx.sm_scale,
                                  bias=ctx.bias, cos=ctx.cos, sin=ctx.sin, rotated=ctx.rotated)
        return None, dQ, dK, dV, None, None, None


class AttnFuseBlockSparseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, block_mask, bias_kind: int):
        from .block_mask import run_block_sparse
        B, H_q, N_q, D = Q.shape
        sm_scale = 1.0 / (D ** 0.5)
        L = torch.empty(B, H_q, N_q, dtype=torch.float32, device=Q.device)
        out = run_block_sparse(Q, K, V, block_mask, sm_scale, bias_kind=bias_kind, save_lse=L)
        ctx.block_mask, ctx.sm_scale, ctx.bias_kind = block_mask, sm_scale, bias_kind
        ctx.save_for_backward(Q, K, V, out, L)
        return out

    @staticmethod
    def backward(ctx, dO):
        from .block_mask import run_block_sparse_backward
        Q, K, V, O, L = ctx.saved_tensors
        dQ, dK, dV = run_block_sparse_backward(Q, K, V, O, L, dO.contiguous(), ctx.block_mask,
                                               ctx.sm_scale, ctx.bias_kind)
        return dQ, dK, dV, None, None
