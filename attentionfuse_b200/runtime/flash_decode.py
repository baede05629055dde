"""Split-K flash-decoding for query length 1.

Mirrors the reference's decode path (attnfuse/runtime/flash_decode.py:46-187): the same
eligibility rule (N_q == 1, N_kv >= 256, dense or ALiBi, no RoPE), fp32 workspaces allocated
per call, a split launch followed by a combine launch.  Extensions: per-sequence valid
lengths (``kv_lens``) and, for KV-sharded multi-GPU decoding, a key offset plus a packed
(normalised O, LSE) partial output.
"""
from __future__ import annotations

import ctypes as C
import functools
from typing import Optional

import torch

from ..ir.high_level import Graph, BiasKind, MaskKind
from . import _lib

_DECODE_TEMPLATES: dict = {}
DECODE_HEAD_DIMS = (64, 128)
DECODE_DTYPES = (torch.float16, torch.bfloat16)


def can_use_flash_decode(graph: Graph, Q: torch.Tensor, K: torch.Tensor, positioned: bool = False) -> bool:
    """The reference's rule (query length 1, N_kv >= 256, dense or ALiBi, no RoPE:
    attnfuse/runtime/flash_decode.py:46-65).  With ``positioned`` -- the caller said where the
    query row sits on the key axis -- causal and sliding-window masks and RoPE are taken too:
    for a single row a mask is a range of keys, and the kernel rotates the row and the key tiles."""
    if Q.shape[2] != 1 or K.shape[2] < 256:
        return False
    allowed_masks = {MaskKind.FULL, MaskKind.CAUSAL, MaskKind.SLIDING_WINDOW} if positioned else {MaskKind.FULL}
    if {m.kind for m in graph.collect_masks()} - allowed_masks:
        return False
    if {b.kind for b in graph.collect_biases()} - {BiasKind.ALIBI}:
        return False
    if graph.has_rope() and not positioned:
        return False
    # The mma.sync decode kernels are instantiated for these types and head dims; anything
    # else takes the general forward kernel (N_q = 1 is a legal dense problem there).
    if Q.dtype not in DECODE_DTYPES or Q.shape[3] not in DECODE_HEAD_DIMS:
        return False
    if K.stride(3) != 1 or Q.stride(3) != 1:
        return False
    if any(s % 8 for s in K.stride()[:3]) or K.data_ptr() % 16:
        return False
    return True


@functools.lru_cache(maxsize=8)
def _sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def _pick_num_splits(B: int, H_q: int, H_kv: int, N_kv: int, device_index: int = 0, ragged: bool = False) -> int:
    """Split count (stands in for attnfuse/runtime/flash_decode.py:69-95)."""
    return int(_lib.load().af_decode_num_splits(B, H_q, H_kv, N_kv, _sm_count(device_index), int(ragged)))


def default_balanced_ctas(B: int, H_q: int, H_kv: int, N_kv: int, device_index: int = 0) -> int:
    """CTAs of the balanced schedule for a problem, or 0 where the split grid stays in charge.
    Groups of up to 16 query heads per KV head (the bandwidth-bound mma.sync kernel): one wave of
    two CTAs per SM, each with at least four 64-key tiles (measured on B16 H32/8 D128 against the
    best split grid: 235 vs 248 us at L = 32768 with ragged lengths, 310 vs 327 us with equal ones,
    47 vs 52 us at L = 4096).  Larger groups (MQA) run on the tensor-core split-K kernel."""
    group = H_q // H_kv
    if group > 16:
        return 0
    tiles = B * H_kv * ((N_kv + 63) // 64)
    return max(1, min(2 * _sm_count(device_index), tiles // 4))


def balanced_rows(B: int, H_q: int, H_kv: int, ctas: int) -> int:
    """Partial rows of the balanced schedule: one slot of min(group, 64) rows per (unit, CTA) pair."""
    group = H_q // H_kv
    units = B * H_kv * ((group + 63) // 64)
    return (units + ctas) * min(group, 64)


def decode_workspace(num_splits: int, B: int, H_q: int, D: int, device, rows: Optional[int] = None):
    """(m, l, acc) partials carved from one allocation.  m and l each take the row count rounded
    up to 4 floats so that acc, which the kernels access with 16-byte vectors, starts on a
    16-byte boundary for every row count.  `rows` overrides num_splits * B * H_q (balanced schedule)."""
    n = num_splits * B * H_q if rows is None else rows
    n_pad = (n + 3) & ~3
    ws = torch.empty(2 * n_pad + n * D, dtype=torch.float32, device=device)
    return ws[:n], ws[n_pad:n_pad + n], ws[2 * n_pad:]


def run_flash_decode(graph: Optional[Graph], Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor,
                     sm_scale: float, bias_kind: int, num_heads_kv: int,
                     out: Optional[torch.Tensor], *, kv_lens: Optional[torch.Tensor] = None,
                     alibi_slopes: Optional[torch.Tensor] = None, kv_offset: int = 0,
                     q_positions: Optional[torch.Tensor] = None,
                     partial: Optional[torch.Tensor] = None,
                     num_splits: Optional[int] = None, workspace=None, exchange=None, exchange_mode: int = 0,
                     mask_kind: int = 0, window: int = 0, q_position: Optional[int] = None,
                     cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                     balanced_ctas: int = 0, kv_rotated: bool = False,
                     kv_pos_block: int = 0, kv_pos_stride: int = 0) -> torch.Tensor:
    """Two launches: split-K partials, then the LSE combine.  Returns `out` (or `partial`
    when only the packed partial is requested)."""
    lib = _lib.load()
    B, H_q, _, D = Q.shape
    _, H_kv, N_kv, _ = K.shape
    if V.stride() != K.stride() and (V.stride(3) != 1 or any(s % 8 for s in V.stride()[:3])):
        V = V.contiguous()
    # A rotated row (cos / sin given) is bound by the rotation of the K tiles, not by bandwidth, and
    # wants the higher occupancy of the split grid (0.60 against 1.2 ms at B16 H32/8 L32768) --
    # unless the cache already holds rotated keys (kv_rotated): then only the query row is rotated.
    if not balanced_ctas and num_splits is None and workspace is None and (cos is None or kv_rotated):
        dev_index = Q.device.index if Q.device.index is not None else torch.cuda.current_device()
        balanced_ctas = default_balanced_ctas(B, H_q, H_kv, N_kv, dev_index)
    if balanced_ctas:
        num_splits = 1
    elif num_splits is None:
        dev_index = Q.device.index if Q.device.index is not None else torch.cuda.current_device()
        num_splits = _pick_num_splits(B, H_q, H_kv, N_kv, dev_index, kv_lens is not None)
    ws_m, ws_l, ws_acc = workspace if workspace is not None else decode_workspace(
        num_splits, B, H_q, D, Q.device, rows=balanced_rows(B, H_q, H_kv, balanced_ctas) if balanced_ctas else None)

    slopes = None
    if bias_kind == 1:
        if alibi_slopes is None:
            from .dispatch import _alibi_slopes
            alibi_slopes = _alibi_slopes(H_q, str(Q.device), str(Q.dtype))
        slopes = alibi_slopes.to(device=Q.device, dtype=Q.dtype).contiguous()
    if kv_lens is not None and (kv_lens.device != Q.device or kv_lens.dtype != torch.int32
                                or not kv_lens.is_contiguous()):
        kv_lens = kv_lens.to(device=Q.device, dtype=torch.int32).contiguous()
    if q_positions is not None and (q_positions.device != Q.device or q_positions.dtype != torch.int32
                                    or not q_positions.is_contiguous()):
        q_positions = q_positions.to(device=Q.device, dtype=torch.int32).contiguous()

    # the shape / stride / flag part of the parameter block is filled once per distinct problem and
    # copied afterwards: a decode step at short caches is bound by this call path
    key = (Q.dtype, Q.shape, Q.stride(), K.shape, K.stride(), V.stride(), None if out is None else out.stride(),
           float(sm_scale), int(bias_kind), int(num_splits), int(kv_offset), int(mask_kind), int(window or 0),
           q_position, cos is not None and cos.stride(0), int(balanced_ctas), bool(kv_rotated),
           int(kv_pos_block), int(kv_pos_stride))
    template = _DECODE_TEMPLATES.get(key)
    if template is None:
        p = _lib.AfDecodeParams()
        p.dtype = _lib.dtype_code(Q.dtype)
        p.B, p.H_q, p.H_kv, p.N_kv, p.D = B, H_q, H_kv, N_kv, D
        p.sm_scale, p.bias_kind, p.num_splits = float(sm_scale), int(bias_kind), int(num_splits)
        p.q_stride, p.k_stride, p.v_stride = _lib.strides(Q), _lib.strides(K), _lib.strides(V)
        p.kv_offset = int(kv_offset)
        p.balanced_ctas = int(balanced_ctas)
        p.kv_pos_block, p.kv_pos_stride = int(kv_pos_block), int(kv_pos_stride)
        p.mask_kind, p.window = int(mask_kind), int(window or 0)
        if q_position is not None:
            p.q_position_p1 = int(q_position) + 1
        if cos is not None:
            p.rope, p.rope_stride_n = (2 if kv_rotated else 1), cos.stride(0)
        if out is not None:
            p.o_stride = _lib.strides(out)
        if len(_DECODE_TEMPLATES) >= 256:
            _DECODE_TEMPLATES.clear()
        template = _DECODE_TEMPLATES[key] = p
    p = _lib.AfDecodeParams.from_buffer_copy(template)
    p.q, p.k, p.v = Q.data_ptr(), K.data_ptr(), V.data_ptr()
    p.slopes, p.kv_lens, p.q_positions = _lib.ptr(slopes), _lib.ptr(kv_lens), _lib.ptr(q_positions)
    if cos is not None:
        p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
    p.ws_m, p.ws_l, p.ws_acc = ws_m.data_ptr(), ws_l.data_ptr(), ws_acc.data_ptr()
    if out is not None:
        p.o = out.data_ptr()
    if partial is not None:
        p.partial = partial.data_ptr()
    with _lib.on_device(Q.device):
        stream = _lib.current_stream(Q.device)
        if exchange is not None and exchange_mode:
            # KV-sharded step in one launch (3), or its push (1) / merge (2) half
            _lib.check(lib.af_decode_sharded_step(C.byref(p), C.byref(exchange.c), int(exchange_mode), stream),
                       "af_decode_sharded_step")
            return out
        _lib.check(lib.af_decode_split(C.byref(p), stream), "af_decode_split")
        if exchange is not None:
            # KV-sharded step: the combine pushes this rank's partial to every rank's exchange
            # buffer; the caller follows up with exchange.wait_merge(out)
            _lib.check(lib.af_decode_combine_push(C.byref(p), C.byref(exchange.c), stream), "af_decode_combine_push")
            return None
        _lib.check(lib.af_decode_combine(C.byref(p), stream), "af_decode_combine")
    return out if out is not None else partial


def combine_gathered(gathered: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Merge per-rank (normalised O, LSE) partials [G, B, H_q, D+1] that live in this GPU's
    own memory into `out` (B, H_q, 1, D)."""
    G, B, H_q, D1 = gathered.shape
    assert gathered.dtype == torch.float32 and gathered.is_contiguous()
    lib = _lib.load()
    with _lib.on_device(out.device):
        rc = lib.af_decode_combine_gathered(gathered.data_ptr(), G, B, H_q, D1 - 1,
                                            _lib.dtype_code(out.dtype), out.data_ptr(),
                                            _lib.strides(out), _lib.current_stream(out.device))
    _lib.check(rc, "af_decode_combine_gathered")
    return out
