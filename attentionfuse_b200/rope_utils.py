"""RoPE tables and the host-side rotate-half application.

Restates attnfuse/rope_utils.py:33-73: theta_i = base^(-2i/D); the table row for position t
is [t*theta_0 .. t*theta_{D/2-1}] repeated twice, so cos/sin have duplicated halves;
apply_rope(x) = x*cos + rotate_half(x)*sin with rotate_half([x1|x2]) = [-x2|x1].
"""
from __future__ import annotations

import torch


def build_rope_cache(seqlen: int, head_dim: int, base: float = 10_000.0,
                     device="cuda", dtype: torch.dtype = torch.float16):
    """Return (cos, sin), each (1, 1, seqlen, head_dim) in ``dtype``."""
    exponent = torch.arange(0, head_dim // 2, device=device, dtype=torch.float32) * 2 / head_dim
    inv_freq = 1.0 / (base ** exponent)
    pos = torch.arange(seqlen, device=device, dtype=torch.float32)
    angle = torch.outer(pos, inv_freq)
    angle = torch.cat([angle, angle], dim=-1)
    return (angle.cos().to(dtype)[None, None], angle.sin().to(dtype)[None, None])


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    lo, hi = x.chunk(2, dim=-1)
    return torch.cat([-hi, lo], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate x (B, H, N, D); cos/sin broadcast from (N, D) or (1, 1, N, D)."""
    return x * cos + _rotate_half(x) * sin
