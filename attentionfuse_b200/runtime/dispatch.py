"""Launch the forward kernel for a graph and real tensors.

Mirrors run_attention of the reference (attnfuse/runtime/dispatch.py:69-215): the same
validation and exception types, the same routing (flash-decoding for query length 1, masked
cross-attention rejected), the same ownership rules (O allocated here unless ``out=`` is
given; ``save_lse`` is a caller-allocated fp32 (B, H_q, N_q) buffer).  The launch itself is
one call into the C-ABI library on torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import functools
import math
import os
from typing import Optional

import torch

from ..ir.high_level import Graph, MaskKind
from . import _lib
from .kernel_cache import get_or_compile


@functools.lru_cache(maxsize=32)
def _alibi_slopes(n_heads: int, device_str: str, dtype_str: str) -> torch.Tensor:
    """ALiBi slopes (Press et al.), created in the requested dtype as the reference does
    (attnfuse/runtime/dispatch.py:24-40): geometric sequence for power-of-two head counts,
    otherwise the closest power of two plus every other slope of the doubled sequence."""
    def geometric(n):
        ratio = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [ratio * (ratio ** i) for i in range(n)]

    if n_heads & (n_heads - 1) == 0:
        values = geometric(n_heads)
    else:
        base = 1 << ((n_heads - 1).bit_length() - 1)
        values = geometric(base) + geometric(2 * base)[0::2][: n_heads - base]
    return torch.tensor(values, dtype=getattr(torch, dtype_str.replace("torch.", "")),
                        device=device_str)


_ROPE_VIEWS: dict = {}


def _rope_table(t: torch.Tensor, name: str, like: torch.Tensor) -> torch.Tensor:
    """The (N, D) view of a cos / sin table in Q's dtype on Q's device; the view of a table seen
    before is remembered (a serving loop passes the same (1, 1, N, D) tables on every call)."""
    key = (t.data_ptr(), t.shape, t.stride(), t.dtype, like.dtype, like.device)
    hit = _ROPE_VIEWS.get(key)
    if hit is not None and hit[0] is t:
        return hit[1]
    view = _rope_table_view(t, name, like)
    if len(_ROPE_VIEWS) >= 16:
        _ROPE_VIEWS.clear()
    _ROPE_VIEWS[key] = (t, view)
    return view


def _rope_table_view(t: torch.Tensor, name: str, like: torch.Tensor) -> torch.Tensor:
    if t.dim() == 4:
        t = t.squeeze(0).squeeze(0)
    if t.dim() != 2:
        raise ValueError(f"{name} must have shape (N, D) or (1, 1, N, D); got {tuple(t.shape)}")
    if t.dtype != like.dtype or t.device != like.device:
        t = t.to(device=like.device, dtype=like.dtype)
    return t if t.stride(1) == 1 else t.contiguous()


def fill_problem(p: _lib.AfProblem, Q, K, V, *, sm_scale, mask_kind, window=0, bias_kind=0,
                 norm_kind=0, slopes=None, bias=None, cos=None, sin=None, family=None, keep=None,
                 q_offset=0):
    """Fill the shape / operand part of a parameter block.  `keep` collects tensors that must
    outlive the launch call (temporaries made contiguous here)."""
    B, H_q, N_q, D = Q.shape
    _, H_kv, N_kv, _ = K.shape
    p.dtype = _lib.dtype_code(Q.dtype)
    if family is None:
        family = int(os.environ.get("ATTNFUSE_FAMILY", "0"))
    p.family = family
    p.B, p.H_q, p.H_kv, p.N_q, p.N_kv, p.D = B, H_q, H_kv, N_q, N_kv, D
    p.sm_scale = float(sm_scale)
    p.q_offset = int(q_offset)
    p.mask_kind, p.window, p.bias_kind, p.norm_kind = mask_kind, int(window or 0), bias_kind, norm_kind
    p.q, p.q_stride = Q.data_ptr(), _lib.strides(Q)
    p.k, p.k_stride = K.data_ptr(), _lib.strides(K)
    p.v, p.v_stride = V.data_ptr(), _lib.strides(V)
    if slopes is not None:
        p.slopes = slopes.data_ptr()
    if bias is not None:
        p.bias, p.bias_stride = bias.data_ptr(), _lib.strides(bias)
    if cos is not None:
        p.rope = 1
        p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
        if cos.stride(0) != sin.stride(0):
            sin = sin.contiguous(); cos = cos.contiguous()
            if keep is not None:
                keep += [cos, sin]
            p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
        p.rope_stride_n = cos.stride(0)


def validate_qkv(Q, K, V):
    if not (Q.is_cuda and K.is_cuda and V.is_cuda):
        raise RuntimeError("AttnFuse requires Q/K/V on a CUDA device.")
    if K.shape != V.shape:
        raise ValueError(f"K and V must have the same shape; got {K.shape}, {V.shape}")
    if Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError(f"Q and K/V must agree on (batch, head_dim); got Q={Q.shape}, K={K.shape}")
    if Q.shape[1] % K.shape[1] != 0:
        raise ValueError(
            f"Q heads ({Q.shape[1]}) must be a multiple of KV heads ({K.shape[1]}) for GQA")
    if not (Q.dtype == K.dtype == V.dtype):
        raise ValueError(f"Q/K/V dtypes differ: {Q.dtype}, {K.dtype}, {V.dtype}")


# Parameter blocks of the forward launch, filled once per (composition, shapes, strides) and copied
# per call: a call then sets only the pointers.  The reference pays its launch path on every call
# (about 40 arguments through the Triton launcher: attnfuse/runtime/dispatch.py:196-214).
_FWD_TEMPLATES: dict = {}
_FWD_TEMPLATES_MAX = 256
# Workspace of forward calls outside autograd (the rotated Q and K of a RoPE problem), kept per
# (device, stream) and grown on demand: calls on one stream are ordered, so they can share it.
_INFER_WORKSPACE: dict = {}


def _inference_workspace(device, stream: int, need: int) -> torch.Tensor:
    key = (device.index, stream)
    ws = _INFER_WORKSPACE.get(key)
    if ws is None or ws.numel() < need:
        ws = _INFER_WORKSPACE[key] = torch.empty(need, dtype=torch.uint8, device=device)
    return ws


def launch_forward(Q, K, V, out, *, sm_scale, mask_kind, window=0, bias_kind=0, norm_kind=0,
                   slopes=None, bias=None, cos=None, sin=None, save_lse=None,
                   block_lists=None, family=None, q_offset=0, keep_workspace=None):
    """Fill AfFwdParams and call af_fwd on the current stream.  `keep_workspace`, a list, receives
    the workspace tensor when the call used one (the rotated Q and K of a RoPE problem, which the
    backward can take over instead of rotating again)."""
    lib = _lib.load()
    if family is None:
        family = int(os.environ.get("ATTNFUSE_FAMILY", "0"))
    in_kernel_rope = os.environ.get("ATTNFUSE_ROPE_IN_KERNEL", "0") == "1"
    key = None
    if block_lists is None and bias is None:
        key = (Q.dtype, Q.shape, Q.stride(), K.shape, K.stride(), V.stride(), out.stride(), float(sm_scale), mask_kind,
               window, bias_kind, norm_kind, family, q_offset, cos is not None and (cos.stride(0), sin.stride(0)),
               save_lse is not None and save_lse.stride(), (Q.data_ptr() | K.data_ptr() | V.data_ptr() | out.data_ptr()) & 15)
        hit = _FWD_TEMPLATES.get(key)
    else:
        hit = None
    if hit is not None:
        template, need = hit
        params = _lib.AfFwdParams.from_buffer_copy(template)
        p = params.p
        p.q, p.k, p.v, params.o = Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr()
        if slopes is not None:
            p.slopes = slopes.data_ptr()
        if cos is not None:
            p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
        if save_lse is not None:
            params.lse = save_lse.data_ptr()
    else:
        params = _lib.AfFwdParams()
        keep: list = []
        fill_problem(params.p, Q, K, V, sm_scale=sm_scale, mask_kind=mask_kind, window=window,
                     bias_kind=bias_kind, norm_kind=norm_kind, slopes=slopes, bias=bias,
                     cos=cos, sin=sin, family=family, keep=keep, q_offset=q_offset)
        if block_lists is not None:
            block_lists.fill(params.p, Q.shape[1])
        params.o, params.o_stride = out.data_ptr(), _lib.strides(out)
        if save_lse is not None:
            params.lse, params.lse_stride = save_lse.data_ptr(), _lib.strides(save_lse, 3)
        need = int(lib.af_fwd_workspace_bytes(C.byref(params)))
        if key is not None and not keep:
            if len(_FWD_TEMPLATES) >= _FWD_TEMPLATES_MAX:
                _FWD_TEMPLATES.clear()
            _FWD_TEMPLATES[key] = (_lib.AfFwdParams.from_buffer_copy(params), need)
    stream = _lib.current_stream(Q.device)
    if need > 0 and not in_kernel_rope:
        if keep_workspace is not None:
            workspace = torch.empty(need, dtype=torch.uint8, device=Q.device)
            keep_workspace.append(workspace)
        else:
            workspace = _inference_workspace(Q.device, stream, need)
        params.workspace, params.workspace_bytes = workspace.data_ptr(), need
    with _lib.on_device(Q.device):
        rc = lib.af_fwd(C.byref(params), stream)
    _lib.check(rc, "af_fwd")
    return out


def run_attention(graph: Graph, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                  bias: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                  sin: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  save_lse: Optional[torch.Tensor] = None, *, alibi_slopes=None,
                  kv_lens: Optional[torch.Tensor] = None, family: Optional[int] = None,
                  q_offset: Optional[int] = None, keep_workspace: Optional[list] = None,
                  kv_rotated: bool = False) -> torch.Tensor:
    """Run the fused forward; returns O with Q's shape and dtype.

    Extensions over the reference signature (all keyword-only): ``alibi_slopes`` overrides the
    default slope table of an ALiBi graph; ``kv_lens`` (int32 [B]) gives per-sequence valid
    cache lengths for query-length-1 decoding; ``family`` forces a kernel family; ``q_offset``
    places query row 0 at that position of the key axis (chunked prefill against a cache: row
    i is masked, biased and rotated as position ``q_offset + i``), which also lifts the
    reference's restriction of masked graphs to N_q == N_kv (attnfuse/runtime/dispatch.py:140-148).
    ``kv_rotated=True`` (positioned single-row decode of a RoPE graph) says that the cache already
    holds rotated keys, as a serving stack stores them: only the query row is rotated, at its
    position, and the step stays bandwidth-bound.  Anywhere else it is refused.
    """
    validate_qkv(Q, K, V)
    N_q, N_kv = Q.shape[2], K.shape[2]
    bundle = get_or_compile(graph)
    q_positions = None
    if isinstance(q_offset, torch.Tensor):
        # per-sequence positions of a single query row (decoding a ragged batch)
        if N_q != 1 or q_offset.shape != (Q.shape[0],):
            raise ValueError("a tensor q_offset gives one position per batch entry and needs query length 1")
        q_positions, q_offset = q_offset, None
    if q_offset is not None and (not isinstance(q_offset, int) or q_offset < 0):
        raise ValueError(f"q_offset must be a non-negative int or an int32 tensor (B,); got {q_offset!r}")

    from .flash_decode import can_use_flash_decode, run_flash_decode
    positioned = q_offset is not None or q_positions is not None
    if save_lse is None and can_use_flash_decode(graph, Q, K, positioned):
        if out is None:
            out = torch.empty_like(Q)
        c = s = None
        if bundle.has_rope:
            if cos is None or sin is None:
                raise RuntimeError(
                    "This attention graph was built with af.rope(); you must pass cos=<table> "
                    "and sin=<table> at call time.")
            c, s = _rope_table(cos, "cos", Q), _rope_table(sin, "sin", Q)
            if c.shape[1] != Q.shape[3] or s.shape != c.shape or c.shape[0] < N_kv or (
                    q_offset is not None and c.shape[0] <= q_offset) or c.stride(0) != s.stride(0):
                raise ValueError(f"cos/sin tables must cover every key and the query position; got {tuple(c.shape)}")
        return run_flash_decode(graph, Q, K, V, bundle.sm_scale, bundle.bias_kind, K.shape[1], out,
                                kv_lens=kv_lens, alibi_slopes=alibi_slopes, q_positions=q_positions,
                                q_position=q_offset, mask_kind=bundle.mask_kind, window=bundle.window,
                                cos=c, sin=s, kv_rotated=kv_rotated)
    if kv_rotated:
        raise ValueError("kv_rotated applies to the positioned single-row decode of a RoPE graph only "
                         "(query length 1 with q_offset, f16/bf16, head_dim 64/128, N_kv >= 256)")
    if q_positions is not None:
        raise ValueError("per-sequence query positions are only supported on the flash-decoding path "
                         "(query length 1, f16/bf16, head_dim 64/128, N_kv >= 256)")
    if kv_lens is not None:
        raise ValueError("kv_lens is only supported on the flash-decoding path "
                         "(query length 1, f16/bf16, head_dim 64/128, N_kv >= 256)")

    if N_q != N_kv and q_offset is None:
        kinds = {m.kind for m in graph.collect_masks()}
        if kinds - {MaskKind.FULL}:
            raise ValueError(
                f"Cross-attention (N_q={N_q} != N_kv={N_kv}) is only supported for full/dense "
                f"masks; the graph uses {sorted(k.value for k in kinds)}. Use "
                "af.softmax(af.scaled_dot_product(Q, K)) @ V for KV-cache decoding.")

    if out is None:
        out = torch.empty_like(Q)

    slopes = None
    if bundle.bias_kind == 1:
        slopes = alibi_slopes if alibi_slopes is not None else _alibi_slopes(
            Q.shape[1], str(Q.device), str(Q.dtype))
        slopes = slopes.to(device=Q.device, dtype=Q.dtype).contiguous()
    if bundle.has_additive_bias:
        if bias is None:
            raise RuntimeError(
                "This attention graph was built with af.additive_bias(); you must pass "
                "bias=<tensor of shape (B,H,N,N)> at call time.")
        if bias.dtype != Q.dtype:
            bias = bias.to(Q.dtype)
    else:
        bias = None
    c = s = None
    if bundle.has_rope:
        if cos is None or sin is None:
            raise RuntimeError(
                "This attention graph was built with af.rope(); you must pass cos=<table> "
                "and sin=<table> at call time.")
        c, s = _rope_table(cos, "cos", Q), _rope_table(sin, "sin", Q)
        if c.shape[0] < max(N_q + (q_offset or 0), N_kv) or c.shape[1] != Q.shape[3] or s.shape != c.shape:
            raise ValueError(f"cos/sin tables must be (>= {max(N_q + (q_offset or 0), N_kv)}, {Q.shape[3]}); "
                             f"got {tuple(c.shape)}, {tuple(s.shape)}")

    return launch_forward(Q, K, V, out, sm_scale=bundle.sm_scale, mask_kind=bundle.mask_kind,
                          window=bundle.window, bias_kind=bundle.bias_kind,
                          norm_kind=bundle.norm_kind, slopes=slopes, bias=bias, cos=c, sin=s,
                          save_lse=save_lse, family=family, q_offset=q_offset or 0,
                          keep_workspace=keep_workspace)
