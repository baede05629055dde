"""Comparison baselines: eager attention and torch SDPA."""
from .pytorch_naive import naive_attention
from .pytorch_sdpa import sdpa_attention

__all__ = ["naive_attention", "sdpa_attention"]
