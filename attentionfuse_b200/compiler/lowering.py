"""Graph -> TiledKernel: fold the combinator chain into one flat record.

Follows the rules of the reference lowering (attnfuse/compiler/lowering.py:20-85):
default scale 1/sqrt(D); {causal, sliding_window} together collapse to the (bidirectional)
sliding window; any other pair of masks, or more than one bias, is not supported.
"""
from __future__ import annotations

import math

from ..ir.high_level import Graph, ScoreKind, MaskKind, NormKind
from ..ir.tiled import TiledKernel
from .fusion import fuse_score_softmax
from .tiling import choose_tile_config


def _fold_masks(masks):
    if not masks:
        return MaskKind.FULL, None
    if len(masks) == 1:
        return masks[0].kind, masks[0].window
    kinds = {m.kind for m in masks}
    if kinds == {MaskKind.CAUSAL, MaskKind.SLIDING_WINDOW}:
        window = [m.window for m in masks if m.kind is MaskKind.SLIDING_WINDOW][0]
        return MaskKind.SLIDING_WINDOW, window
    raise NotImplementedError(f"Mask combination {kinds} not yet supported")


def lower_to_tiled(graph: Graph) -> TiledKernel:
    fuse_score_softmax(graph)
    score = graph.score()
    if score.kind is not ScoreKind.SCALED_DOT:
        raise NotImplementedError(f"Score kind {score.kind} not yet supported")
    D = graph.q.head_dim
    scale = score.scale if score.scale is not None else 1.0 / math.sqrt(D)
    mask_kind, window = _fold_masks(graph.collect_masks())
    biases = graph.collect_biases()
    if len(biases) > 1:
        raise NotImplementedError("Multiple bias ops in one graph not yet supported")
    bias_kind = biases[0].kind if biases else None
    bias_heads = biases[0].num_heads if biases else None
    norm = graph.norm()
    cfg = choose_tile_config(graph)
    if norm.kind is NormKind.RELU:
        cfg.use_streaming_softmax = False
    return TiledKernel(
        head_dim=D, dtype=graph.q.dtype, score_scale=scale,
        mask_kind=mask_kind, mask_window=window,
        bias_kind=bias_kind, bias_num_heads=bias_heads,
        norm_kind=norm.kind, config=cfg,
        rope_kind=1 if score.rope else 0, cache_key=graph.signature())
