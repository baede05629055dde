"""Text renderings of both IR levels (printed under ATTNFUSE_DEBUG=1).

Reference: attnfuse/ir/printer.py:12-83.
"""
from __future__ import annotations

from .high_level import Graph, ScoreOp, MaskOp, BiasOp, NormOp, MatMulPV, TensorSym
from .tiled import TiledKernel


def _sym(t: TensorSym) -> str:
    return f"{t.name}[{t.batch}x{t.num_heads}x{t.seqlen}x{t.head_dim} : {t.dtype}]"


def _render(node, depth: int, out: list, label: str = "") -> None:
    pad = "  " * depth
    head = f"{pad}{label}"
    if isinstance(node, TensorSym):
        out.append(head + _sym(node))
    elif isinstance(node, ScoreOp):
        extra = ", rope" if node.rope else ""
        out.append(head + f"ScoreOp({node.kind.value}, scale={node.scale}{extra})")
        _render(node.q, depth + 1, out, "q = ")
        _render(node.k, depth + 1, out, "k = ")
    elif isinstance(node, MaskOp):
        w = f", window={node.window}" if node.window is not None else ""
        out.append(head + f"MaskOp({node.kind.value}{w})")
        _render(node.scores, depth + 1, out, "scores = ")
    elif isinstance(node, BiasOp):
        h = f", num_heads={node.num_heads}" if node.num_heads is not None else ""
        out.append(head + f"BiasOp({node.kind.value}{h})")
        _render(node.scores, depth + 1, out, "scores = ")
    elif isinstance(node, NormOp):
        out.append(head + f"NormOp({node.kind.value})")
        _render(node.scores, depth + 1, out, "scores = ")
    elif isinstance(node, MatMulPV):
        out.append(head + "MatMulPV")
        _render(node.probs, depth + 1, out, "probs = ")
        _render(node.v, depth + 1, out, "v     = ")
    else:
        out.append(head + repr(node))


def format_graph(g: Graph) -> str:
    lines = [f"# Graph(signature={g.signature()})",
             f"  Q : {_sym(g.q)}", f"  K : {_sym(g.k)}", f"  V : {_sym(g.v)}", "  root:"]
    _render(g.root, 2, lines)
    return "\n".join(lines)


def format_tiled(k: TiledKernel) -> str:
    c = k.config
    mask = k.mask_kind.value + (f" (window={k.mask_window})" if k.mask_window else "")
    bias = (k.bias_kind.value if k.bias_kind else "none") + (
        f" (heads={k.bias_num_heads})" if k.bias_num_heads else "")
    rows = [
        ("dtype", k.dtype), ("head_dim", k.head_dim), ("score_scale", k.score_scale),
        ("mask", mask), ("bias", bias), ("norm", k.norm_kind.value),
        ("rope", k.rope_kind), ("BLOCK_M/BLOCK_N", f"{c.BLOCK_M}/{c.BLOCK_N}"),
        ("num_warps", c.num_warps), ("num_stages", c.num_stages),
    ]
    body = "".join(f"  {name:<15} = {val}\n" for name, val in rows)
    return f"# TiledKernel(cache_key={k.cache_key})\n" + body
