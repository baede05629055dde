"""Gradient parity: dQ, dK, dV from .backward() against torch.autograd through the oracle."""
import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.runtime import _lib
from attentionfuse_b200.runtime.dispatch import _alibi_slopes
from oracle import attention_oracle as orc
from tests._util import assert_close, golden, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"


@af.attention
def dense(Q, K, V):
    return af.softmax(af.scaled_dot_product(Q, K)) @ V


@af.attention
def causal(Q, K, V):
    return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V


@af.attention
def causal_rope(Q, K, V):
    return af.softmax(af.causal(af.rope(Q, K))) @ V


def make_causal_alibi(h):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.causal(af.alibi(af.scaled_dot_product(Q, K), h))) @ V
    return fn


def make_window(w):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), w)) @ V
    return fn


def grads(fn, Q, K, V, dO, **kw):
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (Q, K, V))
    out = fn(q, k, v, **kw)
    out.backward(dO.to(DEV))
    return out, q.grad, k.grad, v.grad


def check(variant, shape, dtype):
    B, Hq, Hkv, N, D = shape
    Q, K, V = qkv(1100, B, Hq, Hkv, N, N, D, dtype)
    dO = orc.randn(1103, (B, Hq, N, D), dtype)
    kw, okw = {}, {"causal": variant.startswith("causal")}
    fn = {"dense": dense, "causal": causal, "causal_rope": causal_rope, "causal_alibi": make_causal_alibi(Hq),
          "window": make_window(23)}[variant]
    if variant == "causal_rope":
        cos, sin = orc.build_rope_cache(N, D, 500000.0, dtype)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV)); okw.update(cos=cos, sin=sin)
    if variant == "causal_alibi":
        okw["slopes"] = _alibi_slopes(Hq, "cpu", str(dtype))
    if variant == "window":
        okw["window"] = 23
    out, dq, dk, dv = grads(fn, Q, K, V, dO, **kw)
    O, dQ, dK, dV = orc.attention_grads(Q, K, V, dO, **okw)
    assert dq.shape == Q.shape and dk.shape == K.shape and dv.shape == V.shape
    assert_close(out, O, dtype, what=f"{variant} O")
    assert_close(dq, dQ, dtype, grad=True, what=f"{variant} dQ")
    assert_close(dk, dK, dtype, grad=True, what=f"{variant} dK")
    assert_close(dv, dV, dtype, grad=True, what=f"{variant} dV")


@pytest.mark.parametrize("variant", ["dense", "causal", "causal_rope", "causal_alibi", "window"])
@pytest.mark.parametrize("shape", [(1, 4, 4, 64, 64), (2, 8, 2, 130, 64), (1, 4, 1, 200, 128), (1, 2, 2, 50, 32)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_backward(variant, shape, dtype):
    check(variant, shape, dtype)


def test_backward_golden():
    g = golden("bwd_small_f32")
    out, dq, dk, dv = grads(causal, g["Q"], g["K"], g["V"], g["dO"])
    assert_close(out, g["O"], torch.float32, what="O")
    assert_close(dq, g["dQ"], torch.float32, grad=True, what="dQ")
    assert_close(dk, g["dK"], torch.float32, grad=True, what="dK")
    assert_close(dv, g["dV"], torch.float32, grad=True, what="dV")
    out, dq, dk, dv = grads(causal_rope, g["Q"], g["K"], g["V"], g["dO"], cos=g["cos"].to(DEV), sin=g["sin"].to(DEV))
    assert_close(out, g["O_rope"], torch.float32, what="O rope")
    assert_close(dq, g["dQ_rope"], torch.float32, grad=True, what="dQ rope")
    assert_close(dk, g["dK_rope"], torch.float32, grad=True, what="dK rope")
    assert_close(dv, g["dV_rope"], torch.float32, grad=True, what="dV rope")


@pytest.mark.parametrize("shape", [(1, 4, 4, 64, 64), (2, 8, 2, 130, 64), (1, 4, 1, 200, 128), (1, 2, 2, 50, 32)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_causal", [False, True], ids=["bias", "causal_bias"])
def test_additive_bias_backward(shape, dtype, with_causal):
    """Gradients of a graph with an additive (B, H, N, N) bias (the reference's can_backward
    excludes it, attnfuse/runtime/backward.py:69-80; here it runs on the exact kernels).  The
    bias itself receives no gradient, as in the reference's autograd contract."""
    B, Hq, Hkv, N, D = shape

    @af.attention
    def fn(Q, K, V):
        s = af.additive_bias(af.scaled_dot_product(Q, K))
        return af.softmax(af.causal(s) if with_causal else s) @ V

    Q, K, V = qkv(1300, B, Hq, Hkv, N, N, D, dtype)
    dO = orc.randn(1303, (B, Hq, N, D), dtype)
    bias = orc.randn(1304, (B, Hq, N, N), dtype)
    out, dq, dk, dv = grads(fn, Q, K, V, dO, bias=bias.to(DEV))
    assert out.requires_grad
    O, dQ, dK, dV = orc.attention_grads(Q, K, V, dO, causal=with_causal, bias=bias.float())
    assert_close(out, O, dtype, what="bias O")
    assert_close(dq, dQ, dtype, grad=True, what="bias dQ")
    assert_close(dk, dK, dtype, grad=True, what="bias dK")
    assert_close(dv, dV, dtype, grad=True, what="bias dV")


def test_no_grad_path_and_unsupported_falls_through():
    Q, K, V = qkv(1200, 1, 2, 2, 64, 64, 64, torch.float16)

    @af.attention
    def relu(Q, K, V):
        return af.relu_attention(af.scaled_dot_product(Q, K)) @ V

    q = Q.to(DEV).requires_grad_(True)
    out = relu(q, K.to(DEV), V.to(DEV))       # no backward for ReLU: inference path, no graph
    assert not out.requires_grad


@pytest.mark.parametrize("variant", ["causal", "causal_rope", "causal_alibi"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_backward_ffma_family_on_half_types(variant, dtype, monkeypatch):
    """The exact FFMA kernels also serve half-precision inputs (forced here); both families must
    meet the same bar."""
    monkeypatch.setenv("ATTNFUSE_FAMILY", "1")
    check(variant, (1, 4, 2, 150, 64), dtype)


@pytest.mark.parametrize("variant", ["dense", "causal", "causal_rope"])
@pytest.mark.parametrize("shape", [(1, 8, 2, 1024, 128), (2, 4, 4, 700, 64), (1, 2, 1, 129, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_backward_tcgen05_longer(variant, shape):
    check(variant, shape, torch.bfloat16)


@pytest.mark.parametrize("variant", ["dense", "causal", "causal_rope", "causal_alibi", "window"])
@pytest.mark.parametrize("shape", [(1, 8, 2, 1024, 128), (2, 2, 1, 333, 128), (1, 4, 4, 64, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_two_pass_and_single_pass_kernels_agree(variant, shape, monkeypatch):
    """Head dim 128 runs the single-pass kernel by default (dQ summed over key tiles in an fp32
    accumulator with atomic adds); ATTNFUSE_BWD_DETERMINISTIC=1 keeps the two-pass kernels.  Both
    meet the bar against the oracle, the two-pass result is bit-reproducible, and the two differ
    by rounding only."""
    B, Hq, Hkv, N, D = shape
    dtype = torch.bfloat16
    Q, K, V = qkv(1500, B, Hq, Hkv, N, N, D, dtype)
    dO = orc.randn(1503, (B, Hq, N, D), dtype)
    kw, okw = {}, {"causal": variant.startswith("causal")}
    fn = {"dense": dense, "causal": causal, "causal_rope": causal_rope, "causal_alibi": make_causal_alibi(Hq),
          "window": make_window(100)}[variant]
    if variant == "causal_rope":
        cos, sin = orc.build_rope_cache(N, D, 500000.0, dtype)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV)); okw.update(cos=cos, sin=sin)
    if variant == "causal_alibi":
        okw["slopes"] = _alibi_slopes(Hq, "cpu", str(dtype))
    if variant == "window":
        okw["window"] = 100
    O, dQ, dK, dV = orc.attention_grads(Q, K, V, dO, **okw)
    before = _lib.launch_count()
    _, dq1, dk1, dv1 = grads(fn, Q, K, V, dO, **kw)
    single_pass_launches = _lib.launch_count() - before
    monkeypatch.setenv("ATTNFUSE_BWD_DETERMINISTIC", "1")
    _, dq2, dk2, dv2 = grads(fn, Q, K, V, dO, **kw)
    _, dq3, dk3, dv3 = grads(fn, Q, K, V, dO, **kw)
    assert torch.equal(dq2, dq3) and torch.equal(dk2, dk3) and torch.equal(dv2, dv3)
    for name, got1, got2, want in (("dQ", dq1, dq2, dQ), ("dK", dk1, dk2, dK), ("dV", dv1, dv2, dV)):
        assert_close(got1, want, dtype, grad=True, what=f"single-pass {variant} {name}")
        assert_close(got2, want, dtype, grad=True, what=f"two-pass {variant} {name}")
        assert orc.rel_fro(got1.float().cpu(), got2.float().cpu()) < 1e-2
    assert single_pass_launches >= 4      # forward (+ rotation), delta, fused pass, dQ finish


@pytest.mark.parametrize("window", [1, 64, 200, 513])
@pytest.mark.parametrize("D", [64, 128])
def test_window_backward_on_tensor_cores(window, D):
    """Sliding-window gradients on the tcgen05 kernels: windows narrower than, equal to and wider
    than the 64-row steps and 128-row stationary tiles, over several tiles, GQA."""
    B, Hq, Hkv, N, dtype = 1, 4, 2, 700, torch.bfloat16
    Q, K, V = qkv(1400 + window, B, Hq, Hkv, N, N, D, dtype)
    dO = orc.randn(1403, (B, Hq, N, D), dtype)
    p = _lib.AfProblem()
    from attentionfuse_b200.runtime.dispatch import fill_problem
    q = Q.to(DEV)
    fill_problem(p, q, K.to(DEV), V.to(DEV), sm_scale=D ** -0.5, mask_kind=2, window=window)
    assert _lib.load().af_query_family(p, 1) == _lib.AF_FAMILY_TCGEN05
    out, dq, dk, dv = grads(make_window(window), Q, K, V, dO)
    O, dQ, dK, dV = orc.attention_grads(Q, K, V, dO, window=window)
    assert_close(out, O, dtype, what="window O")
    assert_close(dq, dQ, dtype, grad=True, what="window dQ")
    assert_close(dk, dK, dtype, grad=True, what="window dK")
    assert_close(dv, dV, dtype, grad=True, what="window dV")
