"""Compiler: combinator graph -> flat kernel record -> key of a pre-built CUDA kernel."""
from .lowering import lower_to_tiled
from .tiling import choose_tile_config
from .fusion import fuse_score_softmax, FusionError
from .codegen import generate_kernel_source, kernel_constexprs
from .variant import VariantKey, variant_for

__all__ = ["lower_to_tiled", "choose_tile_config", "fuse_score_softmax", "FusionError",
           "generate_kernel_source", "kernel_constexprs", "VariantKey", "variant_for"]
