"""Tile selection for sm_100a.

The reference keeps twelve static tables for Ampere/Hopper (attnfuse/compiler/tiling.py:
29-147) and switches on compute capability at import.  This build targets one chip, so
there is one rule: half-precision graphs with head_dim 64 or 128 run on the tcgen05 kernel
whose CTA tile is 128 query rows x 128 keys (the native UMMA M=128 shape, one TMEM lane per
query row); everything else runs on the exact fp32 FFMA kernel with a 32 x 64 tile.
"""
from __future__ import annotations

from ..ir.high_level import Graph, MaskKind
from ..ir.tiled import TileConfig

TC_HEAD_DIMS = (64, 128)
TC_DTYPES = ("float16", "bfloat16")
MAX_HEAD_DIM = 256


def uses_tensor_core_path(head_dim: int, dtype: str) -> bool:
    return head_dim in TC_HEAD_DIMS and dtype in TC_DTYPES


def choose_tile_config(graph: Graph) -> TileConfig:
    if uses_tensor_core_path(graph.q.head_dim, graph.q.dtype):
        cfg = TileConfig(BLOCK_M=128, BLOCK_N=128, num_warps=8, num_stages=2)
    else:
        cfg = TileConfig(BLOCK_M=32, BLOCK_N=64, num_warps=4, num_stages=1)
    if {m.kind for m in graph.collect_masks()} <= {MaskKind.FULL}:
        cfg.skip_full_mask_blocks = False
    return cfg
