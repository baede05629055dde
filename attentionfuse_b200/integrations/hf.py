"""HuggingFace ``attn_implementation="attnfuse"`` backend.

Registers a function in transformers' ALL_ATTENTION_FUNCTIONS on import, as the reference
does (attnfuse/integrations/hf.py:56-145): same signature, SDPA fallback for dropout and for
explicit masks that are not the plain causal triangle, causal graph for prefill and dense
graph (flash-decoding) for query length 1.  Two differences, both required by current
transformers: the result is returned as (B, N, H, D) -- the layout the attention modules
reshape from -- by letting the kernel write through transposed output strides, and the
``scaling`` argument is honoured.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import dsl as _dsl
from ..dsl import api as af

_FN_CACHE: dict = {}


def _get_attn_fn(head_dim: int, dtype: torch.dtype, is_causal: bool, scaling: Optional[float]):
    key = (head_dim, str(dtype), bool(is_causal), None if scaling is None else float(scaling))
    fn = _FN_CACHE.get(key)
    if fn is None:
        if is_causal:
            @af.attention
            def fn(Q, K, V):
                return af.softmax(af.causal(af.scaled_dot_product(Q, K, scale=scaling))) @ V
        else:
            @af.attention
            def fn(Q, K, V):
                return af.softmax(af.scaled_dot_product(Q, K, scale=scaling)) @ V
        _FN_CACHE[key] = fn
    return fn


def _is_pure_causal_mask(mask: Optional[torch.Tensor], N_q: int, N_kv: int) -> bool:
    """True iff `mask` looks like the standard additive causal triangle (-inf above the
    diagonal); checked on the (0, 1) corner only, like the reference (hf.py:105-124)."""
    if mask is None:
        return True
    if mask.dim() != 4 or mask.shape[-2] != N_q or mask.shape[-1] != N_kv:
        return False
    if mask.dtype == torch.bool:
        return N_q == N_kv and N_q > 1 and not bool(mask[..., 0, 1].any().item())
    if N_q > 1 and N_kv > 1:
        corner = mask[..., 0, 1]
        return bool((torch.isinf(corner) | (corner <= torch.finfo(mask.dtype).min / 2)).all().item())
    return True


def _is_chunk_causal_mask(mask: Optional[torch.Tensor], N_q: int, N_kv: int) -> bool:
    """True iff `mask` looks like the causal triangle of a chunk of N_q queries that sits at the
    end of a cache of N_kv keys (row i sees keys 0 .. N_kv - N_q + i): three entries of the
    first row and the last corner are checked, in the spirit of the corner test above."""
    if mask is None or mask.dim() != 4 or mask.shape[-2] != N_q or mask.shape[-1] != N_kv:
        return False
    if not (1 < N_q < N_kv):
        return False
    off = N_kv - N_q
    probe = torch.stack([mask[..., 0, 0], mask[..., 0, off], mask[..., 0, off + 1], mask[..., -1, -1]], dim=-1)
    if mask.dtype == torch.bool:            # True = attend
        seen = probe
    else:
        seen = probe > torch.finfo(mask.dtype).min / 2
    want = torch.tensor([True, True, False, True], device=mask.device)
    return bool((seen == want).all().item())


def _every_key_visible_to_last_row(mask: Optional[torch.Tensor]) -> bool:
    """In a causal triangle (square, or a chunk at the end of a cache, or a single query row) the
    last query row sees every key.  A padded batch masks whole key columns for some rows of the
    batch, which shows up here; such masks must not be replaced by the plain causal rule."""
    if mask is None:
        return True
    last = mask[..., -1, :]
    seen = last if mask.dtype == torch.bool else last > torch.finfo(mask.dtype).min / 2
    return bool(seen.all().item())


def attnfuse_attention_forward(module: torch.nn.Module, query: torch.Tensor, key: torch.Tensor,
                               value: torch.Tensor, attention_mask: Optional[torch.Tensor],
                               dropout: float = 0.0, scaling: Optional[float] = None,
                               is_causal: Optional[bool] = None, **kwargs) -> Tuple[torch.Tensor, None]:
    """query (B, H_q, N_q, D), key/value (B, H_kv, N_kv, D); GQA handled by the kernel (no
    repeat_kv).  Returns (attn_output as (B, N_q, H_q, D), None)."""
    N_q, N_kv = query.shape[2], key.shape[2]
    wants_grad = torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad)
    # a chunk of queries at the end of a cache: causal with a position offset (forward only)
    chunk = dropout == 0.0 and not wants_grad and _is_chunk_causal_mask(attention_mask, N_q, N_kv)
    needs_fallback = not chunk and (dropout > 0.0 or not _is_pure_causal_mask(attention_mask, N_q, N_kv))
    if not chunk and attention_mask is not None and N_q != N_kv and N_q > 1:
        needs_fallback = True
    if is_causal is None:
        is_causal = getattr(module, "is_causal", True)
    # causal without a mask over a rectangular score matrix: the reference raises here
    # (attnfuse/runtime/dispatch.py:140-148); leave the alignment rule to SDPA rather than
    # silently computing dense attention
    if attention_mask is None and bool(is_causal) and 1 < N_q != N_kv:
        needs_fallback = True
    # the corner probes above accept a padded batch's mask; a fully masked key column gives it away
    if not needs_fallback and not _every_key_visible_to_last_row(attention_mask):
        needs_fallback = True
    if needs_fallback:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
        return ALL_ATTENTION_FUNCTIONS["sdpa"](
            module, query, key, value, attention_mask,
            dropout=dropout, scaling=scaling, is_causal=is_causal, **kwargs)

    causal_for_us = chunk or (bool(is_causal) and N_q > 1 and N_q == N_kv)
    attn_fn = _get_attn_fn(query.shape[-1], query.dtype, causal_for_us, scaling)
    B, H, _, D = query.shape
    if wants_grad:
        return attn_fn(query, key, value).transpose(1, 2).contiguous(), None
    # Inference: let the kernel write (B, N, H, D) directly through a transposed view.
    out_bnhd = torch.empty(B, N_q, H, D, dtype=query.dtype, device=query.device)
    from ..runtime.dispatch import run_attention
    graph = attn_fn(query, key, value, return_graph=True)
    run_attention(graph, query, key, value, out=out_bnhd.transpose(1, 2),
                  q_offset=(N_kv - N_q) if chunk else None)
    return out_bnhd, None


def register() -> None:
    """Register the backend; afterwards ``config._attn_implementation = "attnfuse"`` selects it."""
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    except ImportError as e:  # pragma: no cover
        raise ImportError("HuggingFace transformers >= 4.48 is required for this integration") from e
    ALL_ATTENTION_FUNCTIONS["attnfuse"] = attnfuse_attention_forward
    try:  # newer transformers also validate the name against a mask-interface registry
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
        if "attnfuse" not in ALL_MASK_ATTENTION_FUNCTIONS:
            ALL_MASK_ATTENTION_FUNCTIONS["attnfuse"] = ALL_MASK_ATTENTION_FUNCTIONS["sdpa"]
    except Exception:
        pass


register()
