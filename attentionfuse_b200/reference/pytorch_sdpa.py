"""torch SDPA wrapper, a comparison baseline (attnfuse/reference/pytorch_sdpa.py)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sdpa_attention(Q, K, V, *, causal: bool = False, attn_mask=None):
    return F.scaled_dot_product_attention(Q, K, V, attn_mask=attn_mask,
                                          is_causal=causal and attn_mask is None)
