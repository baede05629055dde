"""Multi-GPU work partitioning with no collective: units of (batch, kv head).

A unit is one KV head of one batch row together with the query heads of its group, so the
dK/dV group reduction of the backward stays local to a rank.  Units are numbered
``b * H_kv + h_kv`` and dealt out in contiguous ranges; a range is expressed as at most
three rectangles ``(b_lo, b_hi, h_lo, h_hi)`` so that each piece is a plain slice of the
(B, H, N, D) tensors and of per-head tables (ALiBi slopes, per-head block lists).
The reference is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

from typing import List, Tuple

Rect = Tuple[int, int, int, int]


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced range of units for `rank` (first `n_units % world` ranks get one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def rectangles(B: int, H_kv: int, lo: int, hi: int) -> List[Rect]:
    """Cover units [lo, hi) of a (B, H_kv) grid with at most three rectangles."""
    rects: List[Rect] = []
    if hi <= lo:
        return rects
    b0, h0 = divmod(lo, H_kv)
    b1, h1 = divmod(hi, H_kv)          # exclusive end: (b1, h1)
    if b0 == b1:
        return [(b0, b0 + 1, h0, h1)]
    if h0 != 0:
        rects.append((b0, b0 + 1, h0, H_kv))
        b0 += 1
    if b1 > b0:
        rects.append((b0, b1, 0, H_kv))
    if h1 != 0:
        rects.append((b1, b1 + 1, 0, h1))
    return rects


def shard(B: int, H_kv: int, world: int, rank: int) -> List[Rect]:
    lo, hi = unit_range(B * H_kv, world, rank)
    return rectangles(B, H_kv, lo, hi)


def slice_qkv(Q, K, V, rect: Rect):
    """Views of Q (B, H_q, N, D) and K/V (B, H_kv, N, D) restricted to one rectangle."""
    b_lo, b_hi, h_lo, h_hi = rect
    group = Q.shape[1] // K.shape[1]
    return (Q[b_lo:b_hi, h_lo * group:h_hi * group], K[b_lo:b_hi, h_lo:h_hi], V[b_lo:b_hi, h_lo:h_hi])
