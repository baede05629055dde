"""Two IR levels: the combinator graph and the flat lowered kernel record."""
from .high_level import (
    Expr, TensorSym, ScoreOp, MaskOp, BiasOp, NormOp, MatMulPV, Graph,
    ScoreKind, MaskKind, BiasKind, NormKind,
)
from .tiled import TiledKernel, TileConfig
from .printer import format_graph, format_tiled

__all__ = [
    "Expr", "TensorSym", "ScoreOp", "MaskOp", "BiasOp", "NormOp", "MatMulPV", "Graph",
    "ScoreKind", "MaskKind", "BiasKind", "NormKind",
    "TiledKernel", "TileConfig", "format_graph", "format_tiled",
]
