"""Variant keys: the name of one compile-time specialised kernel instantiation.

The shared library holds explicit C++ template instantiations; lowering a graph yields the
integer codes the C-ABI parameter blocks carry (dtype / mask / bias / norm / rope) plus the
kernel family.  The integer codes are the reference's constexpr encodings
(attnfuse/compiler/codegen.py:17-57: MASK_KIND 0 full, 1 causal, 2 sliding window;
BIAS_KIND 0 none, 1 ALiBi, 2 additive; NORM_KIND 0 softmax, 1 ReLU), extended with
MASK_KIND 3 for block lists.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..ir.high_level import MaskKind, BiasKind, NormKind
from ..ir.tiled import TiledKernel
from .tiling import uses_tensor_core_path

DTYPE_CODE = {"float16": 0, "bfloat16": 1, "float32": 2}
MASK_CODE = {MaskKind.FULL: 0, MaskKind.CAUSAL: 1, MaskKind.SLIDING_WINDOW: 2,
             MaskKind.BLOCK_SPARSE: 3}
BIAS_CODE = {None: 0, BiasKind.ALIBI: 1, BiasKind.ADDITIVE: 2}
NORM_CODE = {NormKind.SOFTMAX: 0, NormKind.RELU: 1}

FAMILY_AUTO, FAMILY_FFMA, FAMILY_TCGEN05 = 0, 1, 2


@dataclass(frozen=True)
class VariantKey:
    op: str            # "fwd" | "decode" | "bwd" | "bs_fwd" | "bs_bwd"
    dtype: int
    head_dim: int
    mask: int
    window: int
    bias: int
    norm: int
    rope: int
    save_lse: int
    family: int

    def name(self) -> str:
        fam = {FAMILY_FFMA: "ffma", FAMILY_TCGEN05: "tcgen05"}.get(self.family, "auto")
        dt = {0: "f16", 1: "bf16", 2: "f32"}[self.dtype]
        return (f"af_{self.op}<{fam},{dt},D{self.head_dim},mask{self.mask},bias{self.bias},"
                f"norm{self.norm},rope{self.rope},lse{self.save_lse}>")


def variant_for(kernel: TiledKernel, op: str = "fwd", save_lse: bool = False) -> VariantKey:
    if kernel.dtype not in DTYPE_CODE:
        raise NotImplementedError(f"dtype {kernel.dtype} has no kernel instantiation")
    tc = (uses_tensor_core_path(kernel.head_dim, kernel.dtype)
          and kernel.norm_kind is NormKind.SOFTMAX
          and kernel.bias_kind is not BiasKind.ADDITIVE)
    return VariantKey(
        op=op, dtype=DTYPE_CODE[kernel.dtype], head_dim=kernel.head_dim,
        mask=MASK_CODE[kernel.mask_kind], window=int(kernel.mask_window or 0),
        bias=BIAS_CODE[kernel.bias_kind], norm=NORM_CODE[kernel.norm_kind],
        rope=int(kernel.rope_kind), save_lse=int(bool(save_lse)),
        family=FAMILY_TCGEN05 if tc else FAMILY_FFMA)
