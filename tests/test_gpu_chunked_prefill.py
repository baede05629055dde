"""Chunked prefill against a cache: a block of N_q query rows placed at position `q_offset` of a
longer key axis (an extension; the reference rejects masked graphs when N_q != N_kv,
attnfuse/runtime/dispatch.py:140-148).  Checked two ways: against the CPU oracle given the same
offset, and against the same rows of the full square problem run through the same kernels."""
import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.runtime import _lib
from attentionfuse_b200.runtime.dispatch import _alibi_slopes
from oracle import attention_oracle as orc
from tests._util import assert_close, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"


def graphs(H, window):
    sdp = af.scaled_dot_product
    return {
        "causal": af.attention(lambda Q, K, V: af.softmax(af.causal(sdp(Q, K))) @ V),
        "window": af.attention(lambda Q, K, V: af.softmax(af.sliding_window(sdp(Q, K), window)) @ V),
        "causal_alibi": af.attention(lambda Q, K, V: af.softmax(af.causal(af.alibi(sdp(Q, K), H))) @ V),
        "causal_rope": af.attention(lambda Q, K, V: af.softmax(af.causal(af.rope(Q, K))) @ V),
        "causal_rope_alibi": af.attention(lambda Q, K, V: af.softmax(af.causal(af.alibi(af.rope(Q, K), H))) @ V),
    }


def oracle_kwargs(variant, H, dtype, window, cos, sin):
    kw = {"causal": variant.startswith("causal")}
    if variant == "window":
        kw["window"] = window
    if "alibi" in variant:
        kw["slopes"] = _alibi_slopes(H, "cpu", str(dtype))
    if "rope" in variant:
        kw.update(cos=cos, sin=sin)
    return kw


@pytest.mark.parametrize("variant", ["causal", "window", "causal_alibi", "causal_rope", "causal_rope_alibi"])
@pytest.mark.parametrize("case", [  # dtype, family, B, H_q, H_kv, N_kv, N_q, q_offset, D
    (torch.bfloat16, _lib.AF_FAMILY_TCGEN05, 2, 8, 2, 700, 200, 500, 128),
    (torch.float16, _lib.AF_FAMILY_TCGEN05, 1, 4, 4, 1000, 130, 611, 64),
    (torch.bfloat16, _lib.AF_FAMILY_TCGEN05, 1, 4, 1, 900, 257, 300, 128),     # cache longer than the last query position
    (torch.float32, _lib.AF_FAMILY_FFMA, 1, 2, 2, 300, 77, 223, 32),
], ids=["bf16-d128", "f16-d64", "bf16-gap", "f32-ffma"])
def test_chunk_matches_oracle_and_full_problem(variant, case):
    dtype, family, B, Hq, Hkv, N_kv, N_q, off, D = case
    window = 150
    Qfull, K, V = qkv(3100 + N_kv, B, Hq, Hkv, N_kv, N_kv, D, dtype)
    Qc = Qfull[:, :, off:off + N_q].contiguous()
    cos, sin = orc.build_rope_cache(N_kv, D, 10000.0, dtype)
    fn = graphs(Hq, window)[variant]
    kw = dict(cos=cos.to(DEV), sin=sin.to(DEV)) if "rope" in variant else {}
    got = fn(Qc.to(DEV), K.to(DEV), V.to(DEV), q_offset=off, family=family, **kw)
    assert got.shape == Qc.shape and got.dtype == dtype
    want = orc.attention(Qc, K, V, q_offset=off, **oracle_kwargs(variant, Hq, dtype, window, cos, sin))
    assert_close(got, want, dtype, what=f"chunk vs oracle {variant}")
    # size-independent property: the chunk is a slice of the square problem
    full = fn(Qfull.to(DEV), K.to(DEV), V.to(DEV), family=family, **kw)
    # fp32 and the one-head tensor-core schedule walk a row in the same order in both problems;
    # in the two-heads-per-CTA schedule a row's fast / classic softmax steps are voted by its warp,
    # whose other rows differ between the two problems, so a result may land one ulp apart.
    ref = full[:, :, off:off + N_q].float()
    half_ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    tol = 1e-5 if dtype == torch.float32 else max(4e-3, half_ulp * ref.abs().max().item())
    assert (got.float() - ref).abs().max().item() <= tol


def test_offsets_are_validated_and_cross_attention_rule_stays():
    B, H, D = 1, 2, 64
    Q, K, V = qkv(3300, B, H, H, 64, 256, D, torch.bfloat16)
    causal = graphs(H, 16)["causal"]
    with pytest.raises(ValueError, match="q_offset"):
        causal(Q.to(DEV), K.to(DEV), V.to(DEV), q_offset=-1)
    with pytest.raises(ValueError, match="Cross-attention"):
        causal(Q.to(DEV), K.to(DEV), V.to(DEV))
    # an offset of zero is a legal chunk: the first 64 rows of the square problem
    got = causal(Q.to(DEV), K.to(DEV), V.to(DEV), q_offset=0)
    assert_close(got, orc.attention(Q, K, V, causal=True, q_offset=0), torch.bfloat16, what="offset 0")
    rope = graphs(H, 16)["causal_rope"]
    cos, sin = orc.build_rope_cache(256, D, 10000.0, torch.bfloat16)
    with pytest.raises(ValueError, match="cos/sin"):
        rope(Q.to(DEV), K.to(DEV), V.to(DEV), cos=cos.to(DEV), sin=sin.to(DEV), q_offset=250)


@pytest.mark.parametrize("variant", ["causal_rope", "causal_rope_alibi", "window"])
def test_single_query_step_with_masks_and_rotation(variant):
    """A decode step (one query row at the end of the cache) through graphs the split-K decode
    path does not take -- rotation, ALiBi with a causal mask, sliding window: the forward kernels
    serve it with the row placed at position N_kv - 1."""
    dtype, B, Hq, Hkv, N_kv, D, window = torch.bfloat16, 2, 8, 2, 1500, 128, 150
    Qfull, K, V = qkv(3500, B, Hq, Hkv, N_kv, N_kv, D, dtype)
    off = N_kv - 1
    Q1 = Qfull[:, :, off:].contiguous()
    cos, sin = orc.build_rope_cache(N_kv, D, 10000.0, dtype)
    fn = graphs(Hq, window)[variant]
    kw = dict(cos=cos.to(DEV), sin=sin.to(DEV)) if "rope" in variant else {}
    got = fn(Q1.to(DEV), K.to(DEV), V.to(DEV), q_offset=off, **kw)
    want = orc.attention(Q1, K, V, q_offset=off, **oracle_kwargs(variant, Hq, dtype, window, cos, sin))
    assert got.shape == (B, Hq, 1, D)
    assert_close(got, want, dtype, what=f"single-row step {variant}")


@pytest.mark.parametrize("case", [(torch.bfloat16, 2, 4, 2, 128), (torch.float16, 1, 4, 4, 64), (torch.bfloat16, 1, 6, 2, 128)],
                         ids=["bf16-d128-pairs", "f16-d64", "bf16-d128-odd-group"])
def test_window_rows_out_of_reach_of_every_key(case):
    """Queries placed past the cache by more than the window see no key at all: whole query tiles
    without a key tile (the persistent kernels skip them in the MMA roles and write zero rows),
    next to tiles that are partly and fully in reach.  Several (batch, head) items per CTA so that
    the barrier phases run across such items."""
    dtype, B, Hq, Hkv, D = case
    N_kv, N_q, off, window = 300, 384, 200, 64
    Q, K, V = qkv(5200, B, Hq, Hkv, N_q, N_kv, D, dtype)
    fn = graphs(Hq, window)["window"]
    got = fn(Q.to(DEV), K.to(DEV), V.to(DEV), q_offset=off, family=_lib.AF_FAMILY_TCGEN05)
    want = orc.attention(Q, K, V, q_offset=off, window=window)
    assert_close(got, want, dtype, what="window past the cache")
    last = got[:, :, N_kv + window - off:].float()
    assert last.numel() > 0 and (last == 0).all()
