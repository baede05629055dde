"""DSL surface, IR helpers and compiler passes on the CPU (no device work)."""
import math

import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.compiler.codegen import kernel_constexprs, generate_kernel_source
from attentionfuse_b200.compiler.fusion import fuse_score_softmax, FusionError
from attentionfuse_b200.compiler.lowering import lower_to_tiled
from attentionfuse_b200.compiler.tiling import choose_tile_config
from attentionfuse_b200.compiler.variant import variant_for, FAMILY_FFMA, FAMILY_TCGEN05
from attentionfuse_b200.ir.high_level import MaskKind, BiasKind, NormKind, NormOp, MatMulPV, Graph
from attentionfuse_b200.ir.printer import format_graph, format_tiled
from attentionfuse_b200.runtime.backward import can_backward


def zeros(D=32, N=16, H=2, dtype=torch.float32):
    z = torch.zeros(1, H, N, D, dtype=dtype)
    return z, z.clone(), z.clone()


def trace(body, **kw):
    fn = af.attention(body)
    return fn(*zeros(**kw), return_graph=True)


def test_graph_shapes_and_signature():
    g = trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V)
    assert g.score().scale is None and g.collect_masks() == [] and g.norm().kind is NormKind.SOFTMAX
    assert len(g.signature()) == 16
    g2 = trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V)
    gc = trace(lambda Q, K, V: af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V)
    assert g.signature() == g2.signature() != gc.signature()
    assert [m.kind for m in gc.collect_masks()] == [MaskKind.CAUSAL]
    # sequence length and batch do not enter the signature, head_dim and dtype do
    assert trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V, N=64).signature() == g.signature()
    assert trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V, D=64).signature() != g.signature()


def test_validation_errors():
    with pytest.raises(ValueError):
        trace(lambda Q, K, V: af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), 0)) @ V)
    with pytest.raises(ValueError):
        trace(lambda Q, K, V: af.softmax(af.alibi(af.scaled_dot_product(Q, K), 0)) @ V)
    with pytest.raises(TypeError, match="value projection"):
        trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)))
    with pytest.raises(TypeError, match="normalisation"):
        trace(lambda Q, K, V: af.causal(af.scaled_dot_product(Q, K)) @ V)
    with pytest.raises(TypeError):
        trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ 3)
    fn = af.attention(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V)
    with pytest.raises(ValueError, match=r"\(B, H, N, D\)"):
        fn(torch.zeros(2, 4, 8), torch.zeros(2, 4, 8), torch.zeros(2, 4, 8), return_graph=True)
    with pytest.raises(ValueError, match="head_dim mismatch"):
        fn(torch.zeros(1, 1, 4, 8), torch.zeros(1, 1, 4, 16), torch.zeros(1, 1, 4, 8), return_graph=True)
    assert fn.graph_fn is not None


def test_lowering_rules():
    g = trace(lambda Q, K, V: af.softmax(af.causal(af.alibi(af.scaled_dot_product(Q, K), 4))) @ V, D=64, H=4)
    k = lower_to_tiled(g)
    assert (k.head_dim, k.mask_kind, k.bias_kind, k.norm_kind) == (64, MaskKind.CAUSAL, BiasKind.ALIBI, NormKind.SOFTMAX)
    assert abs(k.score_scale - 1 / 8) < 1e-9 and k.bias_num_heads == 4 and k.rope_kind == 0
    assert "BLOCK_M" in format_tiled(k) and "MatMulPV" in format_graph(g) and "ScoreOp" in format_graph(g)
    # causal + sliding window folds to the (bidirectional) window, as in the reference
    k = lower_to_tiled(trace(lambda Q, K, V: af.softmax(af.causal(af.sliding_window(af.scaled_dot_product(Q, K), 9))) @ V))
    assert k.mask_kind is MaskKind.SLIDING_WINDOW and k.mask_window == 9
    with pytest.raises(NotImplementedError):
        lower_to_tiled(trace(lambda Q, K, V: af.softmax(af.causal(af.block_sparse(af.scaled_dot_product(Q, K)))) @ V))
    with pytest.raises(NotImplementedError):
        lower_to_tiled(trace(lambda Q, K, V: af.softmax(af.alibi(af.additive_bias(af.scaled_dot_product(Q, K)), 2)) @ V))
    k = lower_to_tiled(trace(lambda Q, K, V: af.relu_attention(af.full(af.rope(Q, K, scale=0.3))) @ V))
    assert k.rope_kind == 1 and k.score_scale == 0.3 and k.norm_kind is NormKind.RELU and k.mask_kind is MaskKind.FULL
    assert not k.config.use_streaming_softmax


def test_fusion_and_tiling_and_variants():
    g = trace(lambda Q, K, V: af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V, D=64)
    assert fuse_score_softmax(g) is g
    bad = Graph(q=g.q, k=g.k, v=g.v, root=MatMulPV(probs=NormOp(kind=NormKind.SOFTMAX, scores=g.q), v=g.v))
    with pytest.raises(FusionError):
        fuse_score_softmax(bad)
    for D in (32, 64, 96, 128, 256):
        cfg = choose_tile_config(trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V, D=D))
        assert cfg.BLOCK_M >= 32 and cfg.BLOCK_N >= 16
    dense16 = lower_to_tiled(trace(lambda Q, K, V: af.softmax(af.scaled_dot_product(Q, K)) @ V, D=64, dtype=torch.float16))
    causal16 = lower_to_tiled(trace(lambda Q, K, V: af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V, D=64, dtype=torch.float16))
    assert kernel_constexprs(dense16)["MASK_KIND"] != kernel_constexprs(causal16)["MASK_KIND"]
    assert variant_for(dense16).family == FAMILY_TCGEN05 and dense16.config.BLOCK_M == 128
    assert variant_for(lower_to_tiled(g)).family == FAMILY_FFMA          # fp32
    assert "tcgen05" in generate_kernel_source(causal16) and generate_kernel_source(causal16) != generate_kernel_source(dense16)


def test_can_backward_scope():
    assert can_backward(trace(lambda Q, K, V: af.softmax(af.causal(af.rope(Q, K))) @ V))
    assert can_backward(trace(lambda Q, K, V: af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), 4)) @ V))
    assert not can_backward(trace(lambda Q, K, V: af.relu_attention(af.scaled_dot_product(Q, K)) @ V))
    assert not can_backward(trace(lambda Q, K, V: af.softmax(af.block_sparse(af.scaled_dot_product(Q, K))) @ V))


def test_reference_package_name_alias():
    import attnfuse
    from attnfuse.ir.high_level import MaskKind as MK
    from attnfuse.runtime.kernel_cache import clear_cache
    assert attnfuse.attention is af.attention and MK is MaskKind
    clear_cache()
