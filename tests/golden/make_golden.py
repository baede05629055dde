"""Generate the golden fixtures in this directory from the REFERENCE project's own code.

Run on a machine that has a checkout of the reference project; point $ATTNFUSE_REF at it:

    python tests/golden/make_golden.py

The reference package is loaded by path under the alias ``attnfuse_ref`` (so that it cannot
be confused with this repository's package) and only its CPU-runnable pieces are executed:
``reference/pytorch_naive.naive_attention``, ``rope_utils.build_rope_cache`` / ``apply_rope``,
``runtime/dispatch._alibi_slopes`` and the pure-Python ``runtime/block_mask.create_block_mask``.
Compositions follow the recipes of the reference's own tests (cited per case).  Outputs are
small .npz files; larger cases store a strided sample plus float64 checksums.
"""
from __future__ import annotations

import importlib.util
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(os.environ.get("ATTNFUSE_REF", Path.home() / "reference"))


def load_reference():
    spec = importlib.util.spec_from_file_location(
        "attnfuse_ref", REF / "attnfuse" / "__init__.py",
        submodule_search_locations=[str(REF / "attnfuse")])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["attnfuse_ref"] = mod
    spec.loader.exec_module(mod)
    import attnfuse_ref.reference.pytorch_naive as naive
    import attnfuse_ref.rope_utils as rope
    import attnfuse_ref.runtime.dispatch as disp
    import attnfuse_ref.runtime.block_mask as bmask
    return naive.naive_attention, rope, disp._alibi_slopes, bmask.create_block_mask


def randn(seed, shape, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)


def expand_kv(t, group):   # tests/test_gqa.py:34-40
    B, H, N, D = t.shape
    return t.unsqueeze(2).expand(B, H, group, N, D).reshape(B, H * group, N, D).contiguous()


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().to(torch.float32).numpy() if v.dtype in (torch.bfloat16, torch.float16) else v.detach().numpy()
        out[k] = v
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(f"wrote {name}.npz ({(HERE / (name + '.npz')).stat().st_size / 1024:.1f} KiB)")


def main():
    naive_attention, rope, ref_slopes, ref_create_block_mask = load_reference()
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- ALiBi slopes for the head counts the configurations use (dispatch.py:24-40)
    save("alibi_slopes", **{f"h{n}": ref_slopes(n, "cpu", "float32") for n in (1, 2, 4, 8, 12, 16, 32, 64)},
         **{f"h{n}_bf16": ref_slopes(n, "cpu", "bfloat16") for n in (12, 32)})

    # ---- RoPE tables (rope_utils.py:33-54)
    c1, s1 = rope.build_rope_cache(64, 64, base=10000.0, device="cpu", dtype=torch.float32)
    c2, s2 = rope.build_rope_cache(32, 128, base=500000.0, device="cpu", dtype=torch.bfloat16)
    save("rope_tables", cos_64x64_b1e4=c1[0, 0], sin_64x64_b1e4=s1[0, 0],
         cos_32x128_b5e5_bf16=c2[0, 0], sin_32x128_b5e5_bf16=s2[0, 0])

    # ---- small forward cases, fp32, inputs stored (tests/test_correctness.py:43-124)
    B, H, N, D = 1, 4, 96, 32
    Q, K, V = randn(11, (B, H, N, D)), randn(12, (B, H, N, D)), randn(13, (B, H, N, D))
    slopes = ref_slopes(H, "cpu", "float32")
    cos, sin = rope.build_rope_cache(N, D, device="cpu", dtype=torch.float32)
    save("fwd_small_f32", Q=Q, K=K, V=V, slopes=slopes, cos=cos[0, 0], sin=sin[0, 0],
         dense=naive_attention(Q, K, V),
         causal=naive_attention(Q, K, V, causal=True),
         window17=naive_attention(Q, K, V, window=17),
         causal_alibi=naive_attention(Q, K, V, causal=True, alibi_slopes=slopes),
         causal_rope=naive_attention(rope.apply_rope(Q, cos, sin), rope.apply_rope(K, cos, sin), V, causal=True),
         causal_rope_alibi=naive_attention(rope.apply_rope(Q, cos, sin), rope.apply_rope(K, cos, sin), V,
                                           causal=True, alibi_slopes=slopes))

    # ---- GQA, non-multiple-of-tile length (tests/test_gqa.py:57-125)
    B, Hq, Hkv, N, D = 1, 4, 2, 130, 64
    Q, K, V = randn(21, (B, Hq, N, D)), randn(22, (B, Hkv, N, D)), randn(23, (B, Hkv, N, D))
    Ke, Ve = expand_kv(K, Hq // Hkv), expand_kv(V, Hq // Hkv)
    cos, sin = rope.build_rope_cache(N, D, device="cpu", dtype=torch.float32)
    save("fwd_gqa_f32", Q=Q, K=K, V=V, cos=cos[0, 0], sin=sin[0, 0],
         causal=naive_attention(Q, Ke, Ve, causal=True),
         causal_rope=naive_attention(rope.apply_rope(Q, cos, sin), rope.apply_rope(Ke, cos, sin), Ve, causal=True))

    # ---- bf16 causal+RoPE through the eager reference in bf16 (test_correctness.py:105-124)
    B, H, N, D = 1, 2, 128, 128
    Q, K, V = (randn(31 + i, (B, H, N, D), torch.bfloat16) for i in range(3))
    cos, sin = rope.build_rope_cache(N, D, base=500000.0, device="cpu", dtype=torch.bfloat16)
    Qr, Kr = rope.apply_rope(Q, cos, sin), rope.apply_rope(K, cos, sin)
    save("fwd_rope_bf16", Q=Q, K=K, V=V, cos=cos[0, 0], sin=sin[0, 0], Q_rot=Qr, K_rot=Kr,
         causal_rope_bf16_eager=naive_attention(Qr, Kr, V, causal=True),
         causal_rope_f32_on_rounded=naive_attention(Qr.float(), Kr.float(), V.float(), causal=True))

    # ---- decode: N_q = 1 against a cache (tests/test_cross_attention.py:54-90)
    B, Hq, Hkv, L, D = 2, 4, 1, 300, 64
    Q, K, V = randn(41, (B, Hq, 1, D)), randn(42, (B, Hkv, L, D)), randn(43, (B, Hkv, L, D))
    full = torch.matmul(torch.softmax(torch.matmul(Q, expand_kv(K, 4).transpose(-2, -1)) / math.sqrt(D), -1),
                        expand_kv(V, 4))
    lens = [211, 300]
    ragged = torch.cat([
        torch.matmul(torch.softmax(torch.matmul(Q[b:b + 1], expand_kv(K[b:b + 1, :, :n], 4).transpose(-2, -1))
                                   / math.sqrt(D), -1), expand_kv(V[b:b + 1, :, :n], 4))
        for b, n in enumerate(lens)])
    save("decode_small_f32", Q=Q, K=K, V=V, kv_lens=np.array(lens, dtype=np.int32), full=full, ragged=ragged)

    # ---- gradients (tests/test_backward.py:61-161): causal GQA, autograd through the reference
    B, Hq, Hkv, N, D = 1, 4, 2, 80, 32
    Q, K, V, dO = randn(51, (B, Hq, N, D)), randn(52, (B, Hkv, N, D)), randn(53, (B, Hkv, N, D)), randn(54, (B, Hq, N, D))
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out = naive_attention(q, expand_kv(k, 2), expand_kv(v, 2), causal=True)
    out.backward(dO)
    cos, sin = rope.build_rope_cache(N, D, device="cpu", dtype=torch.float32)
    q2, k2, v2 = (t.clone().requires_grad_(True) for t in (Q, K, V))
    out2 = naive_attention(rope.apply_rope(q2, cos, sin), expand_kv(rope.apply_rope(k2, cos, sin), 2),
                           expand_kv(v2, 2), causal=True)
    out2.backward(dO)
    save("bwd_small_f32", Q=Q, K=K, V=V, dO=dO, cos=cos[0, 0], sin=sin[0, 0],
         O=out, dQ=q.grad, dK=k.grad, dV=v.grad,
         O_rope=out2, dQ_rope=q2.grad, dK_rope=k2.grad, dV_rope=v2.grad)

    # ---- block masks: the reference builder's lists for the patterns its tests use
    #      (tests/test_block_sparse.py:55-123), plus the element-mask recipe output (:35-40)
    N, BLK = 256, 64

    def bigbird(q, kv):
        qb, kb = q // BLK, kv // BLK
        return (qb == 0) | (kb == 0) | ((qb - kb).abs() <= 1)

    def strided(q, kv):
        return ((q // BLK) + (kv // BLK)) % 2 == 0

    def ragged_pred(q, kv):   # not block aligned: partial tiles get rounded up
        return (q - kv).abs() <= 70

    lists = {}
    for name, fn, n in (("bigbird", bigbird, 256), ("strided", strided, 256), ("ragged", ragged_pred, 200)):
        bm = ref_create_block_mask(fn, n, n, BLK, BLK, device="cpu")
        for f in ("kv_num_blocks", "kv_indices", "full_kv_num", "full_kv_idx", "q_num_blocks", "q_indices"):
            lists[f"{name}_{f}"] = getattr(bm, f)
        lists[f"{name}_n_active"] = np.array(bm.n_active)
    B, H, D = 1, 2, 32
    Q, K, V = randn(61, (B, H, N, D)), randn(62, (B, H, N, D)), randn(63, (B, H, N, D))
    qi = torch.arange(N)[:, None].expand(N, N)
    kj = torch.arange(N)[None, :].expand(N, N)
    S = torch.einsum("bhid,bhjd->bhij", Q, K) / (D ** 0.5)
    S = S.masked_fill(~bigbird(qi, kj), float("-inf"))
    save("block_sparse_small_f32", Q=Q, K=K, V=V, out_bigbird=torch.softmax(S, -1) @ V, **lists)

    # ---- configuration 1 of the benchmark set: fp32 [2,12,512,64], causal + RoPE + ALiBi with
    #      slopes 2^(-8(h+1)/12); store checksums and a strided sample of the output
    B, H, N, D = 2, 12, 512, 64
    Q, K, V = randn(1000, (B, H, N, D)), randn(1001, (B, H, N, D)), randn(1002, (B, H, N, D))
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / 12.0) for h in range(H)], dtype=torch.float32)
    cos, sin = rope.build_rope_cache(N, D, base=10000.0, device="cpu", dtype=torch.float32)
    out = naive_attention(rope.apply_rope(Q, cos, sin), rope.apply_rope(K, cos, sin), V, causal=True,
                          alibi_slopes=slopes)
    save("cfg1_f32", slopes=slopes, out_sample=out[:, :, ::37, :].contiguous(),
         out_sum=np.array(out.double().sum().item()), out_abs_sum=np.array(out.double().abs().sum().item()),
         q_sum=np.array(Q.double().sum().item()), k_sum=np.array(K.double().sum().item()),
         v_sum=np.array(V.double().sum().item()))


if __name__ == "__main__":
    main()
