"""KV-sequence-sharded decode across GPUs: the one multi-GPU path with an exchange step.

Rank r owns keys [r*L/G, (r+1)*L/G) of every (batch, kv head).  Each rank runs the local
split-K decode on its slice and produces a packed partial (normalised O, LSE) of shape
(B, H_q, D+1) fp32; one all-gather (NCCL over NVLink on GPUs) places all partials in every
rank's own memory, and the gathered-combine kernel merges them there.  A rank whose slice
holds no valid key for a row contributes LSE = -inf and is ignored by the merge.
The reference is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def shard_bounds(L: int, world: int, rank: int) -> Tuple[int, int]:
    """Global key range [lo, hi) owned by `rank`; equal slices of ceil(L / world) keys."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    per = (L + world - 1) // world
    lo = min(rank * per, L)
    return lo, min(lo + per, L)


def local_lengths(kv_lens: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Valid keys of each batch row that fall inside [lo, hi): clamp(len - lo, 0, hi - lo)."""
    return (kv_lens.to(torch.int64) - lo).clamp(min=0, max=hi - lo).to(torch.int32)


def _cuda_partial(Q, K_local, V_local, sm_scale, bias_kind, local_lens, kv_offset, q_positions, slopes):
    from .flash_decode import run_flash_decode
    B, H_q, _, D = Q.shape
    partial = torch.empty(B, H_q, D + 1, dtype=torch.float32, device=Q.device)
    run_flash_decode(None, Q, K_local, V_local, sm_scale, bias_kind, K_local.shape[1], None,
                     kv_lens=local_lens, alibi_slopes=slopes, kv_offset=kv_offset,
                     q_positions=q_positions, partial=partial)
    return partial


def _cuda_combine(gathered, out):
    from .flash_decode import combine_gathered
    return combine_gathered(gathered, out)


def sharded_decode(Q: torch.Tensor, K_local: torch.Tensor, V_local: torch.Tensor,
                   kv_lens: Optional[torch.Tensor], L_total: int, rank: int, world: int, *,
                   sm_scale: Optional[float] = None, bias_kind: int = 0, slopes=None,
                   group=None, out: Optional[torch.Tensor] = None,
                   gather_buffer: Optional[torch.Tensor] = None,
                   local_partial: Callable = _cuda_partial, combine: Callable = _cuda_combine,
                   all_gather: Optional[Callable] = None) -> torch.Tensor:
    """Decode one token against a KV cache sharded by sequence.

    Q (B, H_q, 1, D) is replicated; K_local / V_local (B, H_kv, L_local, D) hold this rank's
    key range; kv_lens (B,) are GLOBAL valid lengths (None: all L_total keys valid).
    `local_partial`, `combine` and `all_gather` are injection points for CPU tests of the host
    logic; by default they are the CUDA kernels and torch.distributed.all_gather_into_tensor.
    Raises RuntimeError if a gathered LSE is NaN (a rank produced garbage).
    """
    import torch.distributed as dist
    B, H_q, _, D = Q.shape
    lo, hi = shard_bounds(L_total, world, rank)
    if K_local.shape[2] < hi - lo:
        raise ValueError(f"rank {rank} owns keys [{lo}, {hi}) but K_local holds {K_local.shape[2]}")
    if kv_lens is None:
        kv_lens = torch.full((B,), L_total, dtype=torch.int32, device=Q.device)
    lens_local = local_lengths(kv_lens, lo, hi).to(Q.device)
    q_positions = (kv_lens.to(torch.int32) - 1).to(Q.device) if bias_kind == 1 else None
    if sm_scale is None:
        sm_scale = 1.0 / (D ** 0.5)
    partial = local_partial(Q, K_local, V_local, sm_scale, bias_kind, lens_local, lo, q_positions, slopes)
    if partial.shape != (B, H_q, D + 1):
        raise RuntimeError(f"local partial has shape {tuple(partial.shape)}, expected {(B, H_q, D + 1)}")
    if gather_buffer is None:
        gather_buffer = torch.empty(world, B, H_q, D + 1, dtype=torch.float32, device=partial.device)
    if all_gather is not None:
        all_gather(gather_buffer, partial)
    elif world > 1:
        dist.all_gather_into_tensor(gather_buffer.view(world * B, H_q, D + 1), partial.contiguous(), group=group)
    else:
        gather_buffer[0].copy_(partial)
    if out is None:
        out = torch.empty_like(Q)
    combine(gather_buffer, out)
    return out


def check_gathered(gathered: torch.Tensor) -> None:
    """Host-side sanity check of gathered partials (debug aid; synchronises)."""
    lse = gathered[..., -1]
    if torch.isnan(lse).any():
        bad = torch.isnan(lse).flatten(1).any(1).nonzero().flatten().tolist()
        raise RuntimeError(f"NaN log-sum-exp in the partials of rank(s) {bad}")
