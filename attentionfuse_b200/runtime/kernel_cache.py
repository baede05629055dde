"""Process-local cache of lowered graphs, keyed by graph signature.

Plays the role of the reference's kernel cache (attnfuse/runtime/kernel_cache.py:54-87), but
there is nothing to compile at run time: a cache entry is the lowered record plus the
integer codes the C-ABI parameter block carries.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass

from ..compiler.lowering import lower_to_tiled
from ..compiler.variant import MASK_CODE, BIAS_CODE, NORM_CODE, variant_for
from ..ir.high_level import Graph
from ..ir.tiled import TiledKernel

_lock = threading.Lock()
_cache: dict = {}


@dataclass
class LaunchBundle:
    kernel: TiledKernel
    sm_scale: float
    mask_kind: int
    window: int
    bias_kind: int
    norm_kind: int
    has_additive_bias: bool
    has_rope: bool
    block_m: int


def get_or_compile(graph: Graph) -> LaunchBundle:
    key = graph.signature()
    with _lock:
        hit = _cache.get(key)
        if hit is not None:
            return hit
        kernel = lower_to_tiled(graph)
        if os.environ.get("ATTNFUSE_DEBUG"):
            from ..ir.printer import format_tiled
            print("[AttnFuse] tiled IR:")
            print(format_tiled(kernel))
            print(f"[AttnFuse] kernel instantiation: {variant_for(kernel).name()}")
        bundle = LaunchBundle(
            kernel=kernel, sm_scale=float(kernel.score_scale),
            mask_kind=MASK_CODE[kernel.mask_kind], window=int(kernel.mask_window or 0),
            bias_kind=BIAS_CODE[kernel.bias_kind], norm_kind=NORM_CODE[kernel.norm_kind],
            has_additive_bias=BIAS_CODE[kernel.bias_kind] == 2, has_rope=kernel.rope_kind == 1,
            block_m=kernel.config.BLOCK_M)
        _cache[key] = bundle
        return bundle


def clear_cache() -> None:
    with _lock:
        _cache.clear()
