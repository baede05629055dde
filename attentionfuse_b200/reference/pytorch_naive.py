"""Eager attention that materialises the full score matrix.

Restates the reference oracle (attnfuse/reference/pytorch_naive.py:11-43) so that the
public import path ``<package>.reference.naive_attention`` exists.  Kept in step with the
reference's own file by a unit test that loads that file by path.  Runs on any device; it is
a comparison baseline, never a fallback for the CUDA kernels.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def naive_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *,
                    causal: bool = False, window: Optional[int] = None,
                    alibi_slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Q, K, V: (B, H, N, D) with equal head counts and sequence lengths for masks."""
    H, N, D = Q.shape[1], Q.shape[2], Q.shape[3]
    s = (Q @ K.transpose(-1, -2)) * (1.0 / math.sqrt(D))
    pos = torch.arange(N, device=Q.device)
    rel = pos[:, None] - pos[None, :]
    if alibi_slopes is not None:
        s = s + (-alibi_slopes.view(1, H, 1, 1) * rel.abs().to(Q.dtype))
    if causal:
        s = s.masked_fill(rel < 0, float("-inf"))
    if window is not None:
        s = s.masked_fill(rel.abs() >= window, float("-inf"))
    return torch.softmax(s, dim=-1) @ V
