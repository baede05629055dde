"""Seeded randomised shapes, in the spirit of the reference's Hypothesis suite
(tests/test_fuzz.py:43-49): batch in {1,2,4}, up to 16 query heads with GQA ratios, sequence
lengths 16..512 that are not multiples of any tile size, head dims on both kernel families
(64/128 on the tensor-core kernels, 32/96 on the exact FFMA kernels), windows 8..256, all six
forward compositions and the five with a backward, f16 and bf16, against the CPU oracle.
The draws come from one numpy generator with a fixed seed, so every run sees the same cases."""
import numpy as np
import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.runtime.dispatch import _alibi_slopes
from oracle import attention_oracle as orc
from tests._util import assert_close, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"

FWD_VARIANTS = ["dense", "causal", "window", "causal_alibi", "causal_rope", "causal_rope_alibi"]
BWD_VARIANTS = ["dense", "causal", "window", "causal_alibi", "causal_rope"]


def draw_cases(seed, variants, per_variant):
    rng = np.random.default_rng(seed)
    cases = []
    for variant in variants:
        for i in range(per_variant):
            H_kv = int(rng.choice([1, 2, 3, 4, 8]))
            group = int(rng.choice([g for g in (1, 2, 4, 8) if g * H_kv <= 16]))
            cases.append(dict(
                variant=variant, B=int(rng.choice([1, 2, 4])), H_q=H_kv * group, H_kv=H_kv,
                N=int(rng.integers(16, 513)), D=int(rng.choice([64, 128, 64, 128, 32, 96])),
                W=int(rng.integers(8, 257)), dtype=[torch.float16, torch.bfloat16][int(rng.integers(0, 2))],
                seed=int(rng.integers(1, 1 << 30))))
    return cases


def case_id(c):
    return (f"{c['variant']}-B{c['B']}H{c['H_q']}q{c['H_kv']}kv-N{c['N']}-D{c['D']}-W{c['W']}-"
            f"{str(c['dtype']).replace('torch.', '')}")


def build(c):
    H = c["H_q"]
    w = c["W"]
    v = c["variant"]

    @af.attention
    def fn(Q, K, V):
        s = af.rope(Q, K) if "rope" in v else af.scaled_dot_product(Q, K)
        if "alibi" in v:
            s = af.alibi(s, H)
        if v.startswith("causal"):
            s = af.causal(s)
        if v == "window":
            s = af.sliding_window(s, w)
        return af.softmax(s) @ V
    return fn


def operands(c):
    dt = c["dtype"]
    Q, K, V = qkv(c["seed"], c["B"], c["H_q"], c["H_kv"], c["N"], c["N"], c["D"], dt)
    kw, okw = {}, {"causal": c["variant"].startswith("causal")}
    if "rope" in c["variant"]:
        cos, sin = orc.build_rope_cache(c["N"], c["D"], 10000.0, dt)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV)); okw.update(cos=cos, sin=sin)
    if "alibi" in c["variant"]:
        okw["slopes"] = _alibi_slopes(c["H_q"], "cpu", str(dt))
    if c["variant"] == "window":
        okw["window"] = c["W"]
    return Q, K, V, kw, okw


@pytest.mark.parametrize("c", draw_cases(20260, FWD_VARIANTS, 8), ids=case_id)
def test_random_forward(c):
    Q, K, V, kw, okw = operands(c)
    got = build(c)(Q.to(DEV), K.to(DEV), V.to(DEV), **kw)
    assert_close(got, orc.attention(Q, K, V, **okw), c["dtype"], what=case_id(c))


@pytest.mark.parametrize("c", draw_cases(20261, BWD_VARIANTS, 6), ids=case_id)
def test_random_backward(c):
    Q, K, V, kw, okw = operands(c)
    dO = orc.randn(c["seed"] + 3, Q.shape, c["dtype"])
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (Q, K, V))
    out = build(c)(q, k, v, **kw)
    assert out.requires_grad
    out.backward(dO.to(DEV))
    O, dQ, dK, dV = orc.attention_grads(Q, K, V, dO, **okw)
    assert_close(out, O, c["dtype"], what=case_id(c) + " O")
    assert_close(q.grad, dQ, c["dtype"], grad=True, what=case_id(c) + " dQ")
    assert_close(k.grad, dK, c["dtype"], grad=True, what=case_id(c) + " dK")
    assert_close(v.grad, dV, c["dtype"], grad=True, what=case_id(c) + " dV")
