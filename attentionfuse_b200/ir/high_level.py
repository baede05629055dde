"""Symbolic attention graph built by the combinators.

Mirrors the node vocabulary of the reference IR (attnfuse/ir/high_level.py:49-229):
``TensorSym``, ``ScoreOp``, ``MaskOp``, ``BiasOp``, ``NormOp``, ``MatMulPV`` and the
``Graph`` wrapper with its ``walk / collect_masks / collect_biases / norm / score /
signature`` helpers.  Nothing here touches device memory; the graph is what the
compiler lowers to a key naming one pre-built sm_100a kernel instantiation.
"""
from __future__ import annotations

import enum
import hashlib
from dataclasses import dataclass, field
from typing import Iterator, List, Optional, Tuple


class ScoreKind(enum.Enum):
    SCALED_DOT = "scaled_dot"


class MaskKind(enum.Enum):
    FULL = "full"
    CAUSAL = "causal"
    SLIDING_WINDOW = "sliding_window"
    BLOCK_SPARSE = "block_sparse"


class BiasKind(enum.Enum):
    ADDITIVE = "additive"
    ALIBI = "alibi"


class NormKind(enum.Enum):
    SOFTMAX = "softmax"
    RELU = "relu"


@dataclass
class Expr:
    """Every node derives from Expr so that ``probs @ V`` is captured as MatMulPV."""

    def __matmul__(self, rhs):
        if not isinstance(rhs, TensorSym):
            raise TypeError(
                "Right-hand side of `@` must be the symbolic V tensor; got "
                + type(rhs).__name__)
        return MatMulPV(probs=self, v=rhs)

    def inputs(self) -> list:
        """Upstream nodes, in the order the signature hashes them."""
        return []


@dataclass
class TensorSym(Expr):
    """Placeholder for a (batch, heads, seqlen, head_dim) tensor."""
    name: str
    batch: int
    num_heads: int
    seqlen: int
    head_dim: int
    dtype: str

    @property
    def shape(self) -> Tuple[int, int, int, int]:
        return (self.batch, self.num_heads, self.seqlen, self.head_dim)


@dataclass
class ScoreOp(Expr):
    kind: ScoreKind
    q: TensorSym
    k: TensorSym
    scale: Optional[float] = None   # None means 1/sqrt(head_dim)
    rope: bool = False              # rotate Q and K inside the kernel

    def inputs(self):
        return [self.q, self.k]


@dataclass
class MaskOp(Expr):
    kind: MaskKind
    scores: Expr
    window: Optional[int] = None

    def inputs(self):
        return [self.scores]


@dataclass
class BiasOp(Expr):
    kind: BiasKind
    scores: Expr
    bias: Optional[TensorSym] = None
    num_heads: Optional[int] = None

    def inputs(self):
        return [self.scores] + ([self.bias] if self.bias is not None else [])


@dataclass
class NormOp(Expr):
    kind: NormKind
    scores: Expr

    def inputs(self):
        return [self.scores]


@dataclass
class MatMulPV(Expr):
    probs: Expr
    v: TensorSym

    def inputs(self):
        return [self.probs, self.v]


def _tag(node) -> Optional[str]:
    """One signature token per op node (leaves contribute nothing)."""
    if isinstance(node, ScoreOp):
        return f"score:{node.kind.value}:scale={node.scale}:rope={node.rope}"
    if isinstance(node, MaskOp):
        return f"mask:{node.kind.value}:w={node.window}"
    if isinstance(node, BiasOp):
        return f"bias:{node.kind.value}:h={node.num_heads}"
    if isinstance(node, NormOp):
        return f"norm:{node.kind.value}"
    if isinstance(node, MatMulPV):
        return "matmul_pv"
    return None


@dataclass
class Graph:
    q: TensorSym
    k: TensorSym
    v: TensorSym
    root: MatMulPV
    _signature: Optional[str] = field(default=None, repr=False)

    def walk(self) -> Iterator[tuple]:
        """Pre-order (node, parent) pairs from the root, each node once."""
        visited = set()
        stack = [(self.root, None)]
        while stack:
            node, parent = stack.pop()
            if id(node) in visited:
                continue
            visited.add(id(node))
            yield node, parent
            for child in reversed(node.inputs() if isinstance(node, Expr) else []):
                stack.append((child, node))

    def _of_type(self, cls) -> list:
        return [n for n, _ in self.walk() if isinstance(n, cls)]

    def collect_masks(self) -> List[MaskOp]:
        return self._of_type(MaskOp)

    def collect_biases(self) -> List[BiasOp]:
        return self._of_type(BiasOp)

    def norm(self) -> NormOp:
        found = self._of_type(NormOp)
        if len(found) != 1:
            raise ValueError(
                f"Graph must contain exactly one normalisation op; got {len(found)}")
        return found[0]

    def score(self) -> ScoreOp:
        found = self._of_type(ScoreOp)
        if len(found) != 1:
            raise ValueError(f"Graph must contain exactly one score op; got {len(found)}")
        return found[0]

    def has_rope(self) -> bool:
        return any(s.rope for s in self._of_type(ScoreOp))

    def signature(self) -> str:
        """16-hex-digit key over dtype, head_dim and the op chain; sequence length and
        batch do not enter (reference: attnfuse/ir/high_level.py:183-207)."""
        if self._signature is None:
            tokens = [f"dtype={self.q.dtype}", f"head_dim={self.q.head_dim}"]
            tokens += [t for t in (_tag(n) for n, _ in self.walk()) if t is not None]
            self._signature = hashlib.sha1("|".join(tokens).encode()).hexdigest()[:16]
        return self._signature
