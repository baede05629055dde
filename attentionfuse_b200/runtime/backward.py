"""Backward launch: dQ, dK, dV from (Q, K, V, O, L, dO).

Mirrors run_backward / can_backward of the reference (attnfuse/runtime/backward.py:69-192).
The supported scope is wider: RoPE graphs have a backward here (the reference has none), and
sliding-window and additive-bias graphs run on the exact FFMA kernels.  Gradients have the
shapes of Q, K, V (dK, dV summed over the query-head group); no gradient is produced for
bias, cos or sin.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from ..ir.high_level import Graph, MaskKind, NormKind
from . import _lib
from .dispatch import _alibi_slopes, _rope_table, fill_problem
from .kernel_cache import get_or_compile


def can_backward(graph: Graph) -> bool:
    """True iff the graph has a backward: softmax normalisation and any of the dense /
    causal / sliding-window masks (block-sparse graphs use their own autograd function)."""
    kinds = {m.kind for m in graph.collect_masks()}
    if MaskKind.BLOCK_SPARSE in kinds:
        return False
    try:
        if graph.norm().kind is not NormKind.SOFTMAX:
            return False
        get_or_compile(graph)
    except (NotImplementedError, ValueError, RuntimeError):
        return False
    return True


def launch_backward(Q, K, V, O, L, dO, *, sm_scale, mask_kind, window=0, bias_kind=0, slopes=None,
                    bias=None, cos=None, sin=None, block_lists=None, family=None, rotated=None):
    """`rotated`: the forward's workspace tensor holding the rotated Q and K (RoPE problems), taken
    over instead of running the rotation pre-pass again."""
    lib = _lib.load()
    B, H_q, N_q, D = Q.shape
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    delta = torch.empty(B, H_q, N_q, dtype=torch.float32, device=Q.device)
    params = _lib.AfBwdParams()
    keep: list = []
    fill_problem(params.p, Q, K, V, sm_scale=sm_scale, mask_kind=mask_kind, window=window,
                 bias_kind=bias_kind, slopes=slopes, bias=bias, cos=cos, sin=sin, family=family,
                 keep=keep)
    if block_lists is not None:
        block_lists.fill(params.p, H_q, backward=True)
    params.o, params.o_stride = O.data_ptr(), _lib.strides(O)
    params.d_o, params.do_stride = dO.data_ptr(), _lib.strides(dO)
    params.lse, params.lse_stride = L.data_ptr(), _lib.strides(L, 3)
    params.delta = delta.data_ptr()
    params.dq, params.dq_stride = dQ.data_ptr(), _lib.strides(dQ)
    params.dk, params.dk_stride = dK.data_ptr(), _lib.strides(dK)
    params.dv, params.dv_stride = dV.data_ptr(), _lib.strides(dV)
    need = int(lib.af_bwd_workspace_bytes(C.byref(params)))
    if need > 0:
        if rotated is not None and rotated.numel() >= need and rotated.device == Q.device:
            workspace, params.workspace_holds_rotated = rotated, 1
        else:
            workspace = torch.empty(need, dtype=torch.uint8, device=Q.device)
        params.workspace, params.workspace_bytes = workspace.data_ptr(), need
    # single-pass kernel: dQ is summed over key tiles in an fp32 accumulator (atomic adds, so its
    # last bits vary from run to run); ATTNFUSE_BWD_DETERMINISTIC=1 keeps the two-pass kernels
    if os.environ.get("ATTNFUSE_BWD_DETERMINISTIC", "0") != "1":
        acc_bytes = int(lib.af_bwd_dq_accum_bytes(C.byref(params)))
        if acc_bytes > 0:
            dq_accum = torch.empty(acc_bytes, dtype=torch.uint8, device=Q.device)
            params.dq_accum, params.dq_accum_bytes = dq_accum.data_ptr(), acc_bytes
    with _lib.on_device(Q.device):
        rc = lib.af_bwd(C.byref(params), _lib.current_stream(Q.device))
    _lib.check(rc, "af_bwd")
    return dQ, dK, dV


def run_backward(graph: Graph, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                 O: torch.Tensor, L: torch.Tensor, dO: torch.Tensor, sm_scale: float,
                 bias: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                 sin: Optional[torch.Tensor] = None, alibi_slopes=None, rotated=None):
    """Return (dQ, dK, dV).  `sm_scale` is the scale the forward used."""
    bundle = get_or_compile(graph)
    slopes = None
    if bundle.bias_kind == 1:
        slopes = alibi_slopes if alibi_slopes is not None else _alibi_slopes(
            Q.shape[1], str(Q.device), str(Q.dtype))
        slopes = slopes.to(device=Q.device, dtype=Q.dtype).contiguous()
    if bundle.has_additive_bias and bias is not None and bias.dtype != Q.dtype:
        bias = bias.to(Q.dtype)
    c = s = None
    if bundle.has_rope:
        c, s = _rope_table(cos, "cos", Q), _rope_table(sin, "sin", Q)
    return launch_backward(Q, K, V, O, L, dO, sm_scale=sm_scale, mask_kind=bundle.mask_kind,
                           window=bundle.window, bias_kind=bundle.bias_kind, slopes=slopes,
                           bias=bias if bundle.has_additive_bias else None, cos=c, sin=s, rotated=rotated)
