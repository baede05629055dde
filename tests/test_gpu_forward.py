"""Forward parity on the GPU: every composition through the public DSL (and so through the
C-ABI library) against the CPU oracle on the same seeded inputs."""
import math

import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.rope_utils import build_rope_cache
from attentionfuse_b200.runtime import _lib
from attentionfuse_b200.runtime.dispatch import _alibi_slopes, run_attention
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


def make_window(w):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), w)) @ V
    return fn


def make_causal_alibi(h):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.causal(af.alibi(af.scaled_dot_product(Q, K), h))) @ V
    return fn


@af.attention
def causal_rope(Q, K, V):
    return af.softmax(af.causal(af.rope(Q, K))) @ V


def make_causal_rope_alibi(h):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.causal(af.alibi(af.rope(Q, K), h))) @ V
    return fn


def run_variant(variant, Q, K, V, family, window=37, rope_base=10000.0):
    """Returns (gpu result, oracle result)."""
    H, N, D, dt = Q.shape[1], Q.shape[2], Q.shape[3], Q.dtype
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    kw, okw = {}, {}
    if "rope" in variant:
        cos, sin = orc.build_rope_cache(max(N, K.shape[2]), D, rope_base, dt)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV))
        okw.update(cos=cos, sin=sin)
    if "alibi" in variant:
        okw["slopes"] = _alibi_slopes(H, "cpu", str(dt))
    fn = {"dense": dense, "causal": causal, "window": make_window(window), "causal_alibi": make_causal_alibi(H),
          "causal_rope": causal_rope, "causal_rope_alibi": make_causal_rope_alibi(H)}[variant]
    okw["causal"] = variant.startswith("causal")
    if variant == "window":
        okw["window"] = window
    got = fn(q, k, v, family=family, **kw)
    return got, orc.attention(Q, K, V, **okw)


VARIANTS = ["dense", "causal", "window", "causal_alibi", "causal_rope", "causal_rope_alibi"]
SHAPES = [  # B, H_q, H_kv, N, D
    (1, 4, 4, 128, 64),
    (2, 8, 2, 130, 64),
    (1, 4, 1, 257, 128),
    (2, 2, 2, 384, 128),
]


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tcgen05_forward(variant, shape, dtype):
    B, Hq, Hkv, N, D = shape
    Q, K, V = qkv(100, B, Hq, Hkv, N, N, D, dtype)
    got, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05)
    assert got.dtype == dtype and got.shape == Q.shape
    assert_close(got, want, dtype, what=f"{variant} {shape} {dtype}")


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("shape", [(1, 4, 2, 77, 32), (2, 4, 4, 130, 64), (1, 2, 1, 65, 96), (1, 2, 2, 40, 256)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_ffma_forward(variant, shape, dtype):
    B, Hq, Hkv, N, D = shape
    Q, K, V = qkv(200, B, Hq, Hkv, N, N, D, dtype)
    got, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_FFMA, window=19)
    assert_close(got, want, dtype, what=f"{variant} {shape} {dtype}")


@pytest.mark.parametrize("N", [1, 15, 16, 17, 127, 128, 129, 255, 256, 300])
@pytest.mark.parametrize("D", [64, 128])
def test_tail_lengths(N, D):
    Q, K, V = qkv(300 + N, 1, 2, 1, N, N, D, torch.bfloat16)
    for variant in ("causal", "window", "causal_rope"):
        got, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_AUTO, window=33)
        assert_close(got, want, torch.bfloat16, what=f"{variant} N={N} D={D}")


def test_golden_fp32_variants():
    g = golden("fwd_small_f32")
    Q, K, V = g["Q"].to(DEV), g["K"].to(DEV), g["V"].to(DEV)
    cos, sin = g["cos"].to(DEV), g["sin"].to(DEV)
    H = Q.shape[1]
    assert_close(dense(Q, K, V), g["dense"], torch.float32, what="dense")
    assert_close(causal(Q, K, V), g["causal"], torch.float32, what="causal")
    assert_close(make_window(17)(Q, K, V), g["window17"], torch.float32, what="window")
    assert_close(make_causal_alibi(H)(Q, K, V), g["causal_alibi"], torch.float32, what="alibi")
    assert_close(causal_rope(Q, K, V, cos=cos, sin=sin), g["causal_rope"], torch.float32, what="rope")
    assert_close(make_causal_rope_alibi(H)(Q, K, V, cos=cos, sin=sin), g["causal_rope_alibi"], torch.float32,
                 what="rope+alibi")
    gq = golden("fwd_gqa_f32")
    Q, K, V = gq["Q"].to(DEV), gq["K"].to(DEV), gq["V"].to(DEV)
    assert_close(causal(Q, K, V), gq["causal"], torch.float32, what="gqa causal")
    assert_close(causal_rope(Q, K, V, cos=gq["cos"].to(DEV), sin=gq["sin"].to(DEV)), gq["causal_rope"],
                 torch.float32, what="gqa rope")


def test_golden_bf16_rope():
    g = golden("fwd_rope_bf16")
    Q, K, V = (g[k].to(torch.bfloat16).to(DEV) for k in ("Q", "K", "V"))
    cos, sin = g["cos"].to(torch.bfloat16).to(DEV), g["sin"].to(torch.bfloat16).to(DEV)
    got = causal_rope(Q, K, V, cos=cos, sin=sin)
    assert_close(got, g["causal_rope_f32_on_rounded"], torch.bfloat16, what="bf16 rope vs fp32-on-rounded")


def test_cfg1_golden():
    """fp32 [2,12,512,64] causal + RoPE + ALiBi with explicit slopes 2^(-8(h+1)/12), max-abs 1e-4."""
    g = golden("cfg1_f32")
    B, H, N, D = 2, 12, 512, 64
    Q, K, V = (orc.randn(1000 + i, (B, H, N, D), torch.float32).to(DEV) for i in range(3))
    cos, sin = build_rope_cache(N, D, base=10000.0, device=DEV, dtype=torch.float32)
    fn = make_causal_rope_alibi(H)
    graph = fn(Q, K, V, return_graph=True)
    out = run_attention(graph, Q, K, V, cos=cos, sin=sin, alibi_slopes=g["slopes"].to(DEV))
    assert_close(out[:, :, ::37, :], g["out_sample"], torch.float32, what="cfg1 sample")
    assert abs(out.double().sum().item() - g["out_sum"].item()) < 5e-2


def test_additive_bias_and_relu_and_scale():
    B, H, N, D = 1, 2, 100, 64
    Q, K, V = qkv(400, B, H, H, N, N, D, torch.float16)
    bias = (orc.randn(403, (B, H, N, N), torch.float32) * 0.1).to(torch.float16)

    @af.attention
    def biased(Q, K, V):
        return af.softmax(af.additive_bias(af.scaled_dot_product(Q, K))) @ V

    @af.attention
    def relu(Q, K, V):
        return af.relu_attention(af.causal(af.scaled_dot_product(Q, K))) @ V

    @af.attention
    def scaled(Q, K, V):
        return af.softmax(af.causal(af.scaled_dot_product(Q, K, scale=0.05))) @ V

    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    assert_close(biased(q, k, v, bias=bias.to(DEV)), orc.attention(Q, K, V, bias=bias.float()), torch.float16, what="bias")
    assert_close(relu(q, k, v), orc.attention(Q, K, V, causal=True, relu=True), torch.float16, what="relu")
    assert_close(scaled(q, k, v), orc.attention(Q, K, V, causal=True, scale=0.05), torch.float16, what="scale")
    with pytest.raises(RuntimeError, match="bias"):
        biased(q, k, v)


def test_cross_attention_and_errors():
    Q, K, V = qkv(500, 2, 4, 2, 50, 333, 64, torch.bfloat16)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    assert_close(dense(q, k, v), orc.attention(Q, K, V), torch.bfloat16, what="cross dense")
    with pytest.raises(ValueError, match="Cross-attention"):
        causal(q, k, v)
    with pytest.raises(RuntimeError):
        dense(Q, K, V)                      # CPU tensors
    with pytest.raises(RuntimeError, match="cos"):
        causal_rope(q[:, :, :50], k[:, :, :50], v[:, :, :50])
    with pytest.raises(ValueError):
        dense(q, k, v[:, :, :10])           # K/V shape mismatch
    with pytest.raises(ValueError):
        dense(q[:, :3], k, v)               # H_q % H_kv


def test_strided_inputs_and_bnhd_output():
    """(B, N, H, D) storage viewed as (B, H, N, D), and an output written through transposed strides."""
    B, H, N, D = 2, 4, 200, 64
    Q, K, V = qkv(600, B, H, H, N, N, D, torch.bfloat16)
    q = Q.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    k = K.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    v = V.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    out = torch.empty(B, N, H, D, dtype=torch.bfloat16, device=DEV)
    graph = causal(q, k, v, return_graph=True)
    run_attention(graph, q, k, v, out=out.transpose(1, 2))
    assert_close(out.transpose(1, 2), orc.attention(Q, K, V, causal=True), torch.bfloat16, what="strided")


def test_deterministic_and_no_stray_writes():
    B, H, N, D = 1, 4, 333, 128
    Q, K, V = qkv(700, B, H, 2, N, N, D, torch.bfloat16)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    cos, sin = build_rope_cache(N, D, device=DEV, dtype=torch.bfloat16)
    graph = causal_rope(q, k, v, return_graph=True)
    big = torch.full((B * H * N * D + 2048,), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1024:1024 + B * H * N * D].view(B, H, N, D)
    run_attention(graph, q, k, v, cos=cos, sin=sin, out=out)
    first = out.clone()
    assert torch.isfinite(first).all()
    assert torch.isnan(big[:1024]).all() and torch.isnan(big[-1024:]).all()
    for _ in range(3):
        run_attention(graph, q, k, v, cos=cos, sin=sin, out=out)
        assert torch.equal(out, first)


def test_lse_output():
    B, H, N, D = 1, 2, 150, 64
    for dtype, fam in ((torch.bfloat16, _lib.AF_FAMILY_TCGEN05), (torch.float32, _lib.AF_FAMILY_FFMA)):
        Q, K, V = qkv(800, B, H, H, N, N, D, dtype)
        L = torch.empty(B, H, N, dtype=torch.float32, device=DEV)
        graph = causal(Q.to(DEV), K.to(DEV), V.to(DEV), return_graph=True)
        run_attention(graph, Q.to(DEV), K.to(DEV), V.to(DEV), save_lse=L, family=fam)
        _, want = orc.attention(Q, K, V, causal=True, return_lse=True)
        assert (L.cpu() - want).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rope_prepass_and_in_kernel_rotation_agree(D, dtype, monkeypatch):
    """Long sequences rotate Q and K once in a pre-pass (caller workspace); short ones, or callers
    that pass no workspace, rotate inside the kernel in shared memory.  Same arithmetic, same bits.
    Several query tiles per CTA, so that the persistent pipeline crosses item boundaries."""
    B, Hq, Hkv, N = 3, 16, 4, 1000
    Q, K, V = qkv(900, B, Hq, Hkv, N, N, D, dtype)
    cos, sin = orc.build_rope_cache(N, D, 500000.0, dtype)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    want = orc.attention(Q, K, V, causal=True, cos=cos, sin=sin)
    # The bit-for-bit comparison is between the two rotation schedules of ONE attention schedule:
    # at head dim 128 rotated operands of a GQA problem would otherwise take the two-heads-per-CTA
    # kernel, which the in-kernel rotation does not have (same arithmetic per element, another
    # order of the online-softmax steps).  That kernel is checked against the oracle below.
    monkeypatch.setenv("ATTNFUSE_FWD_PAIR", "0")
    monkeypatch.setenv("ATTNFUSE_ROPE_IN_KERNEL", "0")
    pre = causal_rope(q, k, v, cos=cos.to(DEV), sin=sin.to(DEV))
    monkeypatch.setenv("ATTNFUSE_ROPE_IN_KERNEL", "1")
    fused = causal_rope(q, k, v, cos=cos.to(DEV), sin=sin.to(DEV))
    assert_close(pre, want, dtype, what="pre-pass")
    assert_close(fused, want, dtype, what="in-kernel")
    assert torch.equal(pre, fused)
    monkeypatch.setenv("ATTNFUSE_FWD_PAIR", "1")
    monkeypatch.setenv("ATTNFUSE_ROPE_IN_KERNEL", "0")
    paired = causal_rope(q, k, v, cos=cos.to(DEV), sin=sin.to(DEV))
    assert_close(paired, want, dtype, what="pre-pass, two heads per CTA")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("variant", ["dense", "causal", "causal_alibi"])
def test_row_maximum_jumps_in_late_tiles(variant, dtype):
    """The softmax group forms P against the standing reference maximum and only verifies the
    tile maximum on the side; a tile that raises the maximum by more than the rescale threshold
    must fall back to the classic order (and rescale the accumulator).  Keys grow along the
    sequence, and a few rows see one very large key late."""
    B, Hq, Hkv, N, D = 1, 4, 2, 700, 128
    Q, K, V = qkv(1200, B, Hq, Hkv, N, N, D, dtype)
    ramp = torch.linspace(0.2, 6.0, N).view(1, 1, N, 1)
    K = (K.float() * ramp).to(dtype)
    K[:, :, 650] = (K[:, :, 650].float() * 3).to(dtype)
    got, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05)
    # These rows are one-hot: an output element is a single V element, up to |4| here, where one
    # ulp of bf16 is 1.6e-2 -- the flat 2e-2 of the unit-scale cases is scaled with that magnitude.
    scale = max(1.0, want.abs().max().item() / 2.0)
    assert torch.isfinite(got).all()
    ma, rf = orc.max_abs(got.cpu(), want), orc.rel_fro(got.cpu(), want)
    assert ma <= 2e-2 * scale and rf <= 1e-2, f"late maxima {variant} {dtype}: max-abs {ma:.3e} (scale {scale:.2f}), rel-Frobenius {rf:.3e}"


@pytest.mark.parametrize("variant", ["dense", "causal", "window", "causal_rope"])
def test_more_items_than_sms(variant):
    """One CTA per SM walks several query tiles: phases of the Q / O hand-over and of the K/V
    ring carry across items, including items of different lengths (causal, window)."""
    B, Hq, Hkv, N, D = 3, 16, 4, 1100, 64     # 3*16*9 = 432 query tiles
    Q, K, V = qkv(1300, B, Hq, Hkv, N, N, D, torch.bfloat16)
    got, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05, window=200)
    assert_close(got, want, torch.bfloat16, what=f"persistent {variant}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("variant", ["dense", "causal", "window", "causal_alibi", "causal_rope"])
def test_two_heads_per_cta_schedule(variant, dtype, monkeypatch):
    """At head dim 128 a GQA problem with an even group runs two query heads of a KV group per CTA
    (one K / V load, two S products, a softmax stream per head).  Same arithmetic per element as
    the one-head schedule: both are checked against the oracle, and against each other within
    the half-precision bound.  Several items per CTA, a ragged last tile, groups of 2 and 6."""
    for (B, Hq, Hkv, N) in ((2, 4, 2, 130), (3, 24, 4, 1000), (1, 12, 2, 1333)):
        Q, K, V = qkv(4100 + N, B, Hq, Hkv, N, N, 128, dtype)
        monkeypatch.setenv("ATTNFUSE_FWD_PAIR", "1")
        pair, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05, window=200, rope_base=500000.0)
        monkeypatch.setenv("ATTNFUSE_FWD_PAIR", "0")
        single, _ = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05, window=200, rope_base=500000.0)
        assert_close(pair, want, dtype, what=f"two heads per CTA {variant} {Hq}/{Hkv} N{N}")
        assert_close(single, want, dtype, what=f"one head per CTA {variant} {Hq}/{Hkv} N{N}")
        assert_close(pair, single.cpu().float(), dtype, what=f"two heads vs one head per CTA {variant}")


def test_two_heads_per_cta_lse_and_offset():
    """The LSE rows of the paired schedule and a chunk of queries against a longer cache."""
    B, Hq, Hkv, N, D = 2, 8, 2, 700, 128
    Q, K, V = qkv(4300, B, Hq, Hkv, N, N, D, torch.bfloat16)
    L = torch.empty(B, Hq, N, dtype=torch.float32, device=DEV)
    graph = causal(Q.to(DEV), K.to(DEV), V.to(DEV), return_graph=True)
    out = run_attention(graph, Q.to(DEV), K.to(DEV), V.to(DEV), save_lse=L, family=_lib.AF_FAMILY_TCGEN05)
    want, want_l = orc.attention(Q, K, V, causal=True, return_lse=True)
    assert_close(out, want, torch.bfloat16, what="paired causal")
    assert (L.cpu() - want_l).abs().max().item() < 2e-2
    off, nq = 400, 250
    Qc = Q[:, :, off:off + nq].contiguous()
    got = causal(Qc.to(DEV), K.to(DEV), V.to(DEV), q_offset=off, family=_lib.AF_FAMILY_TCGEN05)
    assert_close(got, orc.attention(Qc, K, V, causal=True, q_offset=off), torch.bfloat16, what="paired chunk")


@pytest.mark.parametrize("variant", ["dense", "causal", "causal_alibi"])
@pytest.mark.parametrize("case", [(3, 12, 4, 700, 128), (2, 8, 2, 900, 128), (3, 6, 6, 700, 64), (2, 6, 2, 520, 128)],
                         ids=lambda c: "x".join(map(str, c)))
def test_item_order_in_l2_sized_chunks(variant, case, monkeypatch):
    """Problems whose K and V exceed the L2 are dealt out in chunks of (batch, head) units, odd
    chunks with their rows of query tiles reversed.  A budget of a quarter megabyte forces many
    chunks on a small problem: same results as the plain order, on both forward schedules (groups
    of 3, 4 and 1 heads: pairs, one head per CTA, head dim 64)."""
    B, Hq, Hkv, N, D = case
    Q, K, V = qkv(6100 + N, B, Hq, Hkv, N, N, D, torch.bfloat16)
    monkeypatch.setenv("ATTNFUSE_L2_KV_MB", "0.25")
    chunked, want = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05)
    monkeypatch.setenv("ATTNFUSE_L2_KV_MB", "1000000")
    plain, _ = run_variant(variant, Q, K, V, _lib.AF_FAMILY_TCGEN05)
    assert_close(chunked, want, torch.bfloat16, what=f"chunked item order {variant}")
    assert torch.equal(chunked, plain)   # the order of the items does not change what an item computes
