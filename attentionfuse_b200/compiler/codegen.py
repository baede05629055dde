"""Kernel specialisation parameters for a lowered kernel.

In the reference this module returns a Triton source string plus ``tl.constexpr`` launch
arguments (attnfuse/compiler/codegen.py:385-412).  Here nothing is generated at run time:
every composition is an explicit instantiation of a C++ template in the shared library, and
``kernel_constexprs`` returns the same specialisation dictionary so that tools comparing
variants keep working.  ``generate_kernel_source`` returns the instantiation's name.
"""
from __future__ import annotations

from ..ir.tiled import TiledKernel
from .variant import MASK_CODE, BIAS_CODE, NORM_CODE, variant_for


def kernel_constexprs(kernel: TiledKernel) -> dict:
    return {
        "HEAD_DIM": kernel.head_dim,
        "BLOCK_M": kernel.config.BLOCK_M,
        "BLOCK_N": kernel.config.BLOCK_N,
        "MASK_KIND": MASK_CODE[kernel.mask_kind],
        "BIAS_KIND": BIAS_CODE[kernel.bias_kind],
        "NORM_KIND": NORM_CODE[kernel.norm_kind],
        "ROPE_KIND": kernel.rope_kind,
        "SKIP_EMPTY": int(kernel.config.skip_full_mask_blocks),
        "WINDOW": kernel.mask_window or 0,
        "SAVE_L": 0,
    }


def kernel_launch_meta(kernel: TiledKernel) -> dict:
    return {"num_warps": kernel.config.num_warps, "num_stages": kernel.config.num_stages}


def generate_kernel_source(kernel: TiledKernel) -> str:
    """Name of the pre-built CUDA instantiation serving this kernel record."""
    return variant_for(kernel).name()


# Import-compatibility alias for callers written against the reference module.
generate_triton_source = generate_kernel_source
