"""The oracle and the package's own eager restatement, pinned to vectors produced by the
reference project's code (tests/golden/make_golden.py)."""
import math

import torch

from oracle import attention_oracle as orc
from tests._util import golden

import attentionfuse_b200 as af
from attentionfuse_b200.reference import naive_attention
from attentionfuse_b200.rope_utils import build_rope_cache, apply_rope
from attentionfuse_b200.runtime.dispatch import _alibi_slopes

TOL = 2e-6


def close(a, b, tol=TOL):
    assert a.shape == b.shape
    assert (a.double() - b.double()).abs().max().item() <= tol, (a.double() - b.double()).abs().max().item()


def test_alibi_slopes_match_reference():
    g = golden("alibi_slopes")
    for n in (1, 2, 4, 8, 12, 16, 32, 64):
        close(orc.alibi_slopes(n).float(), g[f"h{n}"], 0.0)
        close(_alibi_slopes(n, "cpu", "float32"), g[f"h{n}"], 0.0)
    for n in (12, 32):
        close(_alibi_slopes(n, "cpu", "bfloat16").float(), g[f"h{n}_bf16"], 0.0)
        close(orc.alibi_slopes(n).to(torch.bfloat16).float(), g[f"h{n}_bf16"], 0.0)


def test_rope_tables_match_reference():
    g = golden("rope_tables")
    c, s = orc.build_rope_cache(64, 64, 10000.0)
    close(c, g["cos_64x64_b1e4"], 0.0); close(s, g["sin_64x64_b1e4"], 0.0)
    c, s = build_rope_cache(64, 64, base=10000.0, device="cpu", dtype=torch.float32)
    close(c[0, 0], g["cos_64x64_b1e4"], 0.0); close(s[0, 0], g["sin_64x64_b1e4"], 0.0)
    c, s = orc.build_rope_cache(32, 128, 500000.0, torch.bfloat16)
    close(c.float(), g["cos_32x128_b5e5_bf16"], 0.0); close(s.float(), g["sin_32x128_b5e5_bf16"], 0.0)
    c, s = build_rope_cache(32, 128, base=500000.0, device="cpu", dtype=torch.bfloat16)
    close(c[0, 0].float(), g["cos_32x128_b5e5_bf16"], 0.0)


def test_forward_variants_match_reference():
    g = golden("fwd_small_f32")
    Q, K, V = g["Q"], g["K"], g["V"]
    close(orc.attention(Q, K, V), g["dense"])
    close(orc.attention(Q, K, V, causal=True), g["causal"])
    close(orc.attention(Q, K, V, window=17), g["window17"])
    close(orc.attention(Q, K, V, causal=True, slopes=g["slopes"]), g["causal_alibi"])
    close(orc.attention(Q, K, V, causal=True, cos=g["cos"], sin=g["sin"]), g["causal_rope"])
    close(orc.attention(Q, K, V, causal=True, cos=g["cos"], sin=g["sin"], slopes=g["slopes"]),
          g["causal_rope_alibi"])
    # the package's public eager functions
    close(naive_attention(Q, K, V), g["dense"])
    close(naive_attention(Q, K, V, causal=True), g["causal"])
    close(naive_attention(Q, K, V, window=17), g["window17"])
    close(naive_attention(Q, K, V, causal=True, alibi_slopes=g["slopes"]), g["causal_alibi"])
    close(naive_attention(apply_rope(Q, g["cos"], g["sin"]), apply_rope(K, g["cos"], g["sin"]), V, causal=True),
          g["causal_rope"])


def test_gqa_matches_reference():
    g = golden("fwd_gqa_f32")
    close(orc.attention(g["Q"], g["K"], g["V"], causal=True), g["causal"])
    close(orc.attention(g["Q"], g["K"], g["V"], causal=True, cos=g["cos"], sin=g["sin"]), g["causal_rope"])
    close(orc.attention_chunked(g["Q"], g["K"], g["V"], causal=True), g["causal"])


def test_bf16_rope_rounding_point_matches_reference():
    g = golden("fwd_rope_bf16")
    Q, K, V = (g[k].to(torch.bfloat16) for k in ("Q", "K", "V"))
    cos, sin = g["cos"].to(torch.bfloat16), g["sin"].to(torch.bfloat16)
    # rotated operands as the eager bf16 reference produces them
    got_q = orc.apply_rope(Q.float(), cos.float(), sin.float()).to(torch.bfloat16).float()
    # eager bf16 rounds each product; the oracle rotates in fp32 and rounds once: <= 1 bf16 ulp apart
    assert (got_q - g["Q_rot"]).abs().max().item() <= 2 ** -5
    want = g["causal_rope_f32_on_rounded"]
    got = orc.attention(Q, K, V, causal=True, cos=cos, sin=sin)
    assert orc.rel_fro(got, want) < 5e-3 and orc.max_abs(got, want) < 2e-2
    assert orc.rel_fro(got, g["causal_rope_bf16_eager"]) < 1e-2


def test_decode_matches_reference():
    g = golden("decode_small_f32")
    close(orc.attention(g["Q"], g["K"], g["V"]), g["full"])
    close(orc.attention(g["Q"], g["K"], g["V"], kv_lens=g["kv_lens"]), g["ragged"])


def test_gradients_match_reference():
    g = golden("bwd_small_f32")
    O, dQ, dK, dV = orc.attention_grads(g["Q"], g["K"], g["V"], g["dO"], causal=True)
    close(O, g["O"]); close(dQ, g["dQ"], 1e-5); close(dK, g["dK"], 1e-5); close(dV, g["dV"], 1e-5)
    O, dQ, dK, dV = orc.attention_grads(g["Q"], g["K"], g["V"], g["dO"], causal=True, cos=g["cos"], sin=g["sin"])
    close(O, g["O_rope"]); close(dQ, g["dQ_rope"], 1e-5); close(dK, g["dK_rope"], 1e-5)
    close(dV, g["dV_rope"], 1e-5)


def test_block_sparse_matches_reference():
    g = golden("block_sparse_small_f32")
    bm = af.create_block_mask(lambda q, k: ((q // 64) == 0) | ((k // 64) == 0) | ((q // 64 - k // 64).abs() <= 1),
                              256, 256, 64, 64, device="cpu")
    mask = orc.block_elem_mask(bm.dense_grid(), 64, 64, 256, 256)
    close(orc.attention(g["Q"], g["K"], g["V"], elem_mask=mask), g["out_bigbird"])


def test_cfg1_matches_reference():
    """Configuration 1: fp32 [2,12,512,64], causal + RoPE(base 1e4) + ALiBi slopes 2^(-8(h+1)/12)."""
    g = golden("cfg1_f32")
    B, H, N, D = 2, 12, 512, 64
    Q, K, V = orc.randn(1000, (B, H, N, D), torch.float32), orc.randn(1001, (B, H, N, D), torch.float32), \
        orc.randn(1002, (B, H, N, D), torch.float32)
    assert abs(Q.double().sum().item() - g["q_sum"].item()) < 1e-6, "CPU generator stream changed"
    cos, sin = orc.build_rope_cache(N, D, 10000.0)
    out = orc.attention(Q, K, V, causal=True, cos=cos, sin=sin, slopes=g["slopes"])
    close(out[:, :, ::37, :], g["out_sample"], 5e-6)
    assert abs(out.double().sum().item() - g["out_sum"].item()) < 1e-2


def test_query_offset_rows_are_rows_of_the_square_problem():
    """`q_offset` (chunked prefill against a cache) is defined by this property."""
    from tests._util import qkv
    B, H, N, D, off, n = 1, 3, 96, 16, 40, 30
    Q, K, V = qkv(77, B, H, H, N, N, D, torch.float32)
    cos, sin = orc.build_rope_cache(N, D, 10000.0, torch.float32)
    for kw in (dict(causal=True), dict(window=17), dict(causal=True, slopes=orc.alibi_slopes(H).float()),
               dict(causal=True, cos=cos, sin=sin)):
        full = orc.attention(Q, K, V, **kw)
        part = orc.attention(Q[:, :, off:off + n], K, V, q_offset=off, **kw)
        assert (full[:, :, off:off + n] - part).abs().max().item() < 1e-6
