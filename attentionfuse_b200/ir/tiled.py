"""Flat, lowered description of one fused attention kernel.

Same record the reference's lowering produces (attnfuse/ir/tiled.py:33-81); here the
record is not fed to a code generator but hashed into the key of a compile-time
specialised CUDA instantiation (see compiler/variant.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .high_level import MaskKind, BiasKind, NormKind


@dataclass
class TileConfig:
    """CTA tile of the sm_100a kernel chosen for a graph."""
    BLOCK_M: int = 128
    BLOCK_N: int = 128
    num_warps: int = 8
    num_stages: int = 2
    use_streaming_softmax: bool = True
    skip_full_mask_blocks: bool = True


@dataclass
class TiledKernel:
    head_dim: int
    dtype: str
    score_scale: Optional[float]
    mask_kind: MaskKind = MaskKind.FULL
    mask_window: Optional[int] = None
    bias_kind: Optional[BiasKind] = None
    bias_num_heads: Optional[int] = None
    norm_kind: NormKind = NormKind.SOFTMAX
    config: TileConfig = field(default_factory=TileConfig)
    rope_kind: int = 0
    cache_key: str = ""
