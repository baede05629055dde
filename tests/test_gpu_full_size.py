"""The benchmark configurations at full size.  The CPU oracle checks a slice of each problem
(one batch row / kv-head group, so the score matrix stays small) and size-independent
properties cover the rest: rows of P sum to one (V = 1 gives O = 1), linearity in V, the first
causal row copies V[0], decode results do not depend on the split count."""
import numpy as np
import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.runtime.dispatch import _alibi_slopes
from attentionfuse_b200.runtime.flash_decode import run_flash_decode
from oracle import attention_oracle as orc
from tests._util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gpu_randn(seed, shape, dtype):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=DEV, dtype=dtype)


@af.attention
def dense(Q, K, V):
    return af.softmax(af.scaled_dot_product(Q, K)) @ V


@af.attention
def causal(Q, K, V):
    return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V


@af.attention
def causal_rope(Q, K, V):
    return af.softmax(af.causal(af.rope(Q, K))) @ V


@af.attention
def window256(Q, K, V):
    return af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), 256)) @ V


@af.attention
def causal_alibi12(Q, K, V):
    return af.softmax(af.causal(af.alibi(af.scaled_dot_product(Q, K), 12))) @ V


@af.attention
def causal_rope_alibi12(Q, K, V):
    return af.softmax(af.causal(af.alibi(af.rope(Q, K), 12))) @ V


@af.attention
def bs_attn(Q, K, V):
    return af.softmax(af.block_sparse(af.scaled_dot_product(Q, K))) @ V


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("variant", ["dense", "causal", "window", "causal_alibi", "causal_rope", "causal_rope_alibi"])
def test_cfg2_n4096(variant, dtype):
    """GPT-2/BERT geometry [4,12,4096,64]: oracle on batch row 0, heads 0..2."""
    B, H, N, D = 4, 12, 4096, 64
    Q, K, V = (gpu_randn(2000 + i, (B, H, N, D), dtype) for i in range(3))
    cos, sin = orc.build_rope_cache(N, D, 10000.0, dtype)
    fn = {"dense": dense, "causal": causal, "window": window256, "causal_alibi": causal_alibi12,
          "causal_rope": causal_rope, "causal_rope_alibi": causal_rope_alibi12}[variant]
    kw = dict(cos=cos.to(DEV), sin=sin.to(DEV)) if "rope" in variant else {}
    out = fn(Q, K, V, **kw)
    hs = slice(0, 3)
    okw = dict(causal=variant.startswith("causal"))
    if variant == "window":
        okw["window"] = 256
    if "rope" in variant:
        okw.update(cos=cos, sin=sin)
    if "alibi" in variant:
        okw["slopes"] = _alibi_slopes(H, "cpu", str(dtype))[hs]
    want = orc.attention(Q[:1, hs].cpu(), K[:1, hs].cpu(), V[:1, hs].cpu(), **okw)
    assert_close(out[:1, hs], want, dtype, what=f"cfg2 {variant}")
    # every row of P sums to one
    ones = fn(Q, K, torch.ones_like(V), **kw)
    assert (ones.float() - 1).abs().max().item() < 1e-2
    if variant.startswith("causal"):
        assert torch.equal(out[:, :, 0], V[:, :, 0])          # first causal row sees only key 0


def test_cfg4_forward_backward():
    """Llama-3-8B layer shape, causal + RoPE(5e5), bf16: oracle autograd on one (batch, kv head) group."""
    B, Hq, Hkv, N, D = 4, 32, 8, 4096, 128
    dt = torch.bfloat16
    Q, K, V, dO = (gpu_randn(4000 + i, (B, h, N, D), dt) for i, h in enumerate((Hq, Hkv, Hkv, Hq)))
    cos, sin = orc.build_rope_cache(N, D, 500000.0, dt)
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out = causal_rope(q, k, v, cos=cos.to(DEV), sin=sin.to(DEV))
    out.backward(dO)
    b, g = 2, 5
    hs = slice(4 * g, 4 * g + 4)
    O, dQ, dK, dV = orc.attention_grads(Q[b:b + 1, hs].cpu(), K[b:b + 1, g:g + 1].cpu(), V[b:b + 1, g:g + 1].cpu(),
                                        dO[b:b + 1, hs].cpu(), causal=True, cos=cos, sin=sin)
    assert_close(out[b:b + 1, hs], O, dt, what="cfg4 O")
    assert_close(q.grad[b:b + 1, hs], dQ, dt, grad=True, what="cfg4 dQ")
    assert_close(k.grad[b:b + 1, g:g + 1], dK, dt, grad=True, what="cfg4 dK")
    assert_close(v.grad[b:b + 1, g:g + 1], dV, dt, grad=True, what="cfg4 dV")
    # linearity of the backward in dO: grads(2 dO) = 2 grads(dO)
    q2, k2, v2 = (t.clone().requires_grad_(True) for t in (Q, K, V))
    causal_rope(q2, k2, v2, cos=cos.to(DEV), sin=sin.to(DEV)).backward(2 * dO)
    for a, c in ((q.grad, q2.grad), (k.grad, k2.grad), (v.grad, v2.grad)):
        assert orc.rel_fro(c.float().cpu(), 2 * a.float().cpu()) < 1e-2
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all() and torch.isfinite(v.grad).all()


def test_cfg4_forward_whole_tensor():
    """Llama-3-8B layer shape forward, causal + RoPE(5e5), bf16: every one of the 32 (batch, kv
    head) groups against the oracle (chunked, so the score matrix stays at one group)."""
    B, Hq, Hkv, N, D = 4, 32, 8, 4096, 128
    dt = torch.bfloat16
    Q, K, V = (gpu_randn(4100 + i, (B, h, N, D), dt) for i, h in enumerate((Hq, Hkv, Hkv)))
    cos, sin = orc.build_rope_cache(N, D, 500000.0, dt)
    out = causal_rope(Q, K, V, cos=cos.to(DEV), sin=sin.to(DEV))
    want = orc.attention_chunked(Q.cpu(), K.cpu(), V.cpu(), causal=True, cos=cos, sin=sin)
    assert_close(out, want, dt, what="cfg4 forward, all 32 groups")


@pytest.mark.parametrize("heads", [(32, 8), (64, 8), (64, 1)], ids=lambda h: f"{h[0]}q{h[1]}kv")
@pytest.mark.parametrize("L", [16384, 32768])
def test_cfg3_decode(heads, L):
    """Decode, batch 16, lengths U[L/2, L]: oracle on two batch rows; split count must not matter."""
    Hq, Hkv = heads
    B, D, dt = 16, 128, torch.bfloat16
    Q = gpu_randn(3000, (B, Hq, 1, D), dt)
    K, V = gpu_randn(3001, (B, Hkv, L, D), dt), gpu_randn(3002, (B, Hkv, L, D), dt)
    g = torch.Generator(device="cpu").manual_seed(3000)
    lens = torch.randint(L // 2, L + 1, (B,), generator=g, dtype=torch.int32)
    out = dense(Q, K, V, kv_lens=lens.to(DEV))
    for b in (0, 11):
        want = orc.attention(Q[b:b + 1].cpu(), K[b:b + 1].cpu(), V[b:b + 1].cpu(), kv_lens=lens[b:b + 1])
        assert_close(out[b:b + 1], want, dt, what=f"cfg3 row {b}")
    other = torch.empty_like(out)
    run_flash_decode(None, Q, K, V, 1.0 / D ** 0.5, 0, Hkv, other, kv_lens=lens.to(DEV), num_splits=5)
    assert orc.rel_fro(other.float().cpu(), out.float().cpu()) < 5e-3   # two roundings to bf16
    # keys past the valid length must not matter
    K2, V2 = K.clone(), V.clone()
    for b in range(B):
        K2[b, :, lens[b]:] = 1e4
        V2[b, :, lens[b]:] = float("nan")
    assert torch.equal(dense(Q, K2, V2, kv_lens=lens.to(DEV)), out)


def test_cfg5_bigbird_per_head():
    """fp16 [2,16,8192,64], block 128, per-head BigBird masks, forward + backward, plus the dense control."""
    B, H, N, D, blk = 2, 16, 8192, 64, 128
    nb = N // blk
    dt = torch.float16

    def grid_for(h):
        rng = np.random.default_rng(5000 + h)
        gm = np.zeros((nb, nb), dtype=bool)
        gm[:, :2] = True
        gm[:2, :] = True
        for i in range(nb):
            gm[i, max(0, i - 1):min(nb, i + 2)] = True
            free = np.flatnonzero(~gm[i])
            if len(free):
                gm[i, rng.choice(free, size=min(3, len(free)), replace=False)] = True
        return torch.from_numpy(gm)

    grids = torch.stack([grid_for(h) for h in range(H)])
    bm = af.create_block_mask_per_head(grids, blk, blk, device=DEV)
    assert bm.n_active == int(grids.sum())
    Q, K, V, dO = (gpu_randn(5000 + i, (B, H, N, D), dt) for i in range(4))
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out = bs_attn(q, k, v, block_mask=bm)
    out.backward(dO)
    for h in (0, 9):
        mask = orc.block_elem_mask(grids[h], blk, blk, N, N)
        O, dQ, dK, dV = orc.attention_grads(Q[1:2, h:h + 1].cpu(), K[1:2, h:h + 1].cpu(), V[1:2, h:h + 1].cpu(),
                                            dO[1:2, h:h + 1].cpu(), elem_mask=mask)
        assert_close(out[1:2, h:h + 1], O, dt, what=f"cfg5 O head {h}")
        assert_close(q.grad[1:2, h:h + 1], dQ, dt, grad=True, what=f"cfg5 dQ head {h}")
        assert_close(k.grad[1:2, h:h + 1], dK, dt, grad=True, what=f"cfg5 dK head {h}")
        assert_close(v.grad[1:2, h:h + 1], dV, dt, grad=True, what=f"cfg5 dV head {h}")
    # control: an all-active mask equals dense attention
    full = af.BlockMask.from_dense(torch.ones(nb, nb, dtype=torch.bool), blk, blk, device=DEV)
    assert orc.rel_fro(bs_attn(Q, K, V, block_mask=full).float().cpu(), dense(Q, K, V).float().cpu()) < 2e-3


@pytest.mark.parametrize("variant", ["causal_rope", "window"])
def test_long_sequence_chunks_agree_with_the_whole(variant):
    """A 16k-token problem: the last query chunk run on its own against the full key axis
    (`q_offset`) equals the same rows of the whole problem, the oracle checks those rows, and
    every row of P sums to one (V = 1 gives O = 1)."""
    B, Hq, Hkv, N, D, dtype = 1, 8, 2, 16384, 128, torch.bfloat16
    Q, K, V = gpu_randn(9100, (B, Hq, N, D), dtype), gpu_randn(9101, (B, Hkv, N, D), dtype), gpu_randn(9102, (B, Hkv, N, D), dtype)
    cos, sin = orc.build_rope_cache(N, D, 500000.0, dtype)
    fn, kw, okw = (causal_rope, dict(cos=cos.to(DEV), sin=sin.to(DEV)), dict(causal=True, cos=cos, sin=sin)) \
        if variant == "causal_rope" else (window256, {}, dict(window=256))
    whole = fn(Q, K, V, **kw)
    n_q, off = 384, N - 384
    chunk = fn(Q[:, :, off:].contiguous(), K, V, q_offset=off, **kw)
    assert (chunk.float() - whole[:, :, off:].float()).abs().max().item() <= 4e-3
    want = orc.attention(Q[:, :, off:].cpu(), K.cpu(), V.cpu(), q_offset=off, **okw)
    assert_close(chunk, want, dtype, what=f"16k {variant} chunk")
    ones = fn(Q, K, torch.ones_like(V), **kw)
    assert (ones.float() - 1).abs().max().item() < 1e-2
