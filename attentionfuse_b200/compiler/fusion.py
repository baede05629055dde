"""Shape check for the fusable chain  norm <- (mask | bias)* <- score  under ``@ V``.

Reference: attnfuse/compiler/fusion.py:28-56.  Recognition only; a graph that does not
have this shape cannot be served by a single online-softmax kernel and is rejected.
"""
from __future__ import annotations

from ..ir.high_level import Graph, ScoreOp, MaskOp, BiasOp, NormOp, MatMulPV, NormKind


class FusionError(RuntimeError):
    pass


def fuse_score_softmax(graph: Graph) -> Graph:
    root = graph.root
    if not isinstance(root, MatMulPV):
        raise FusionError("Graph root must be MatMulPV (probs @ V).")
    norm = root.probs
    if not isinstance(norm, NormOp):
        raise FusionError("MatMulPV.probs must be the output of a normalisation combinator.")
    if norm.kind not in (NormKind.SOFTMAX, NormKind.RELU):
        raise FusionError(f"Unsupported normalisation: {norm.kind}")
    node = norm.scores
    while isinstance(node, (MaskOp, BiasOp)):
        node = node.scores
    if not isinstance(node, ScoreOp):
        raise FusionError(
            "Expected the chain norm <- (mask|bias)* <- score; "
            f"hit {type(node).__name__} instead.")
    return graph
