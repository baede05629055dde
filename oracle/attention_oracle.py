"""CPU oracle for the fused-attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain eager PyTorch on the CPU, the arithmetic the reference project
defines for attention; it exists so that tests, the smoke check and the benchmark's
``cpu_baseline`` leg can check and time against it.  Nothing in the product package imports
it, and it is never a fallback for the CUDA kernels.

Each function cites the reference file:line it follows.  The restatement is pinned: the
fixtures under tests/golden/ were produced by running the reference's own functions
(loaded by path from the reference checkout by tests/golden/make_golden.py) and
tests/test_oracle.py checks this file against them.

Precision policy: inputs arrive already rounded to the configuration's dtype (f16 / bf16 /
f32); the oracle up-casts them to fp32 (or fp64 on request) and computes there, so that the
comparison measures the kernel's error, not the eager low-precision path's.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------------------
# building blocks
# ----------------------------------------------------------------------------------------
def alibi_slopes(n_heads: int) -> torch.Tensor:
    """fp64 ALiBi slopes; attnfuse/runtime/dispatch.py:24-40 (the caller rounds them to the
    input dtype, as the reference creates the tensor in Q's dtype)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if n_heads & (n_heads - 1) == 0:
        vals = pow2(n_heads)
    else:
        closest = 1 << ((n_heads - 1).bit_length() - 1)
        vals = pow2(closest) + pow2(2 * closest)[0::2][: n_heads - closest]
    return torch.tensor(vals, dtype=torch.float64)


def build_rope_cache(seqlen: int, head_dim: int, base: float = 10000.0,
                     dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """(cos, sin) of shape (seqlen, head_dim), halves duplicated; attnfuse/rope_utils.py:33-54."""
    half = head_dim // 2
    theta = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) * 2 / head_dim))
    freqs = torch.outer(torch.arange(seqlen, dtype=torch.float32), theta)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin with rotate_half([x1|x2]) = [-x2|x1]; attnfuse/rope_utils.py:57-73."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


def expand_kv(t: torch.Tensor, group: int) -> torch.Tensor:
    """Repeat each KV head `group` times (the reference tests' _expand_kv, tests/test_gqa.py:34-40)."""
    B, H, N, D = t.shape
    return t.unsqueeze(2).expand(B, H, group, N, D).reshape(B, H * group, N, D)


def scores(Q, K, *, scale=None, causal=False, window=None, slopes=None, bias=None,
           elem_mask=None, kv_lens=None, q_positions=None, q_offset=0) -> torch.Tensor:
    """Masked, biased score matrix (B, H, N_q, N_kv) in Q's dtype.

    Follows attnfuse/reference/pytorch_naive.py:22-40 (scale, ALiBi as -slope*|i-j|, causal
    tril, |i-j| < window), plus the additive bias of the reference kernel
    (attnfuse/compiler/codegen.py:347-352), an element mask (tests/test_block_sparse.py:35-40)
    and per-sequence valid lengths for decoding.  `q_positions` (B,) overrides the query
    position used by ALiBi when N_q == 1 (attnfuse/compiler/codegen_decode.py:142-145 measures
    the distance from the last key).  `q_offset` places query row 0 at that position of the key
    axis (chunked prefill against a cache; an extension with no counterpart in the reference,
    defined so that the rows agree with the same rows of the full square problem)."""
    B, H, N_q, D = Q.shape
    N_kv = K.shape[2]
    s = torch.matmul(Q, K.transpose(-2, -1)) * (scale if scale is not None else 1.0 / math.sqrt(D))
    qi = torch.arange(N_q) + q_offset
    kj = torch.arange(N_kv)
    rel = qi[:, None] - kj[None, :]
    if slopes is not None:
        if N_q == 1 and N_kv != 1:
            qpos = (q_positions if q_positions is not None else
                    (kv_lens - 1 if kv_lens is not None else torch.full((B,), N_kv - 1)))
            dist = (qpos.view(B, 1, 1, 1) - kj.view(1, 1, 1, N_kv)).abs().to(Q.dtype)
        else:
            dist = rel.abs().to(Q.dtype).view(1, 1, N_q, N_kv)
        s = s + (-slopes.to(Q.dtype).view(1, H, 1, 1) * dist)
    if bias is not None:
        s = s + bias.to(Q.dtype)
    if causal:
        s = s.masked_fill(rel < 0, float("-inf"))
    if window is not None:
        s = s.masked_fill(rel.abs() >= window, float("-inf"))
    if elem_mask is not None:
        s = s.masked_fill(~elem_mask, float("-inf"))
    if kv_lens is not None:
        dead = kj.view(1, 1, 1, N_kv) >= kv_lens.view(B, 1, 1, 1)
        s = s.masked_fill(dead, float("-inf"))
    return s


def attention(Q, K, V, *, scale=None, causal=False, window=None, slopes=None, bias=None,
              cos=None, sin=None, elem_mask=None, kv_lens=None, q_positions=None,
              relu=False, return_lse=False, dtype=torch.float32, q_offset=0):
    """Full attention in `dtype` with GQA expansion and optional RoPE pre-rotation.

    RoPE: rotate in `dtype`, round the rotated Q, K back to the input dtype, as the reference
    kernel does before its dot (attnfuse/compiler/codegen.py:133-135, 339-341) and as
    apply_rope on low-precision tensors does (tests/test_correctness.py:119-122).
    Rows without any visible key give 0 (the kernel's l == 0 -> 1 rule,
    attnfuse/compiler/codegen.py:370-371), not NaN."""
    in_dtype = Q.dtype
    group = Q.shape[1] // K.shape[1]
    q, k, v = Q.to(dtype), K.to(dtype), V.to(dtype)
    if cos is not None:
        c, s_ = cos.to(dtype), sin.to(dtype)
        q = apply_rope(q, c[q_offset: q_offset + q.shape[2]], s_[q_offset: q_offset + q.shape[2]]).to(in_dtype).to(dtype)
        k = apply_rope(k, c[: k.shape[2]], s_[: k.shape[2]]).to(in_dtype).to(dtype)
    if group > 1:
        k, v = expand_kv(k, group), expand_kv(v, group)
    s = scores(q, k, scale=scale, causal=causal, window=window,
               slopes=None if slopes is None else slopes.to(dtype), bias=bias,
               elem_mask=elem_mask, kv_lens=kv_lens, q_positions=q_positions, q_offset=q_offset)
    if relu:
        # ReLU normalisation: max(s, 0) divided by its row sum (attnfuse/compiler/codegen.py:364-374)
        p = torch.clamp(s, min=0.0)
        l = p.sum(-1, keepdim=True)
        out = torch.matmul(p, v) / torch.where(l == 0, torch.ones_like(l), l)
        return (out, None) if return_lse else out
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse).unsqueeze(-1))
    p = torch.where(torch.isinf(lse).unsqueeze(-1), torch.zeros_like(p), p)
    out = torch.matmul(p, v)
    return (out, lse) if return_lse else out


def attention_chunked(Q, K, V, *, per_head_mask: Optional[Callable] = None, **kw):
    """Same as `attention`, one (batch, kv head) group at a time so the score matrix stays
    small (Cfg-4/5-sized problems).  `per_head_mask(h)` may supply an element mask per head."""
    B, H_q = Q.shape[0], Q.shape[1]
    H_kv = K.shape[1]
    group = H_q // H_kv
    out = torch.empty(Q.shape, dtype=kw.get("dtype", torch.float32))
    slopes = kw.pop("slopes", None)
    bias = kw.pop("bias", None)
    kv_lens = kw.pop("kv_lens", None)
    for b in range(B):
        for g in range(H_kv):
            hs = slice(g * group, (g + 1) * group)
            for h in range(g * group, (g + 1) * group) if per_head_mask else [None]:
                sl = hs if h is None else slice(h, h + 1)
                out[b:b + 1, sl] = attention(
                    Q[b:b + 1, sl], K[b:b + 1, g:g + 1], V[b:b + 1, g:g + 1],
                    slopes=None if slopes is None else slopes[sl],
                    bias=None if bias is None else bias[b:b + 1, sl],
                    kv_lens=None if kv_lens is None else kv_lens[b:b + 1],
                    elem_mask=per_head_mask(h) if h is not None else kw.get("elem_mask"),
                    **{k_: v_ for k_, v_ in kw.items() if k_ != "elem_mask"})
    return out


def attention_grads(Q, K, V, dO, **kw):
    """(O, dQ, dK, dV) by torch.autograd through `attention` in fp32, the recipe of the
    reference's backward tests (tests/test_backward.py:70-73, GQA grads summed over the group
    by autograd through the expansion, :143-158)."""
    dtype = kw.pop("dtype", torch.float32)
    q = Q.to(dtype).detach().requires_grad_(True)
    k = K.to(dtype).detach().requires_grad_(True)
    v = V.to(dtype).detach().requires_grad_(True)
    in_dtype = Q.dtype
    cos, sin = kw.pop("cos", None), kw.pop("sin", None)
    qq, kk = q, k
    if cos is not None:
        # straight-through rounding: the rotated operands are rounded to the input dtype for the
        # matmul, and the gradient flows through the rotation itself
        c, s_ = cos.to(dtype), sin.to(dtype)
        rq = apply_rope(q, c[: q.shape[2]], s_[: q.shape[2]])
        rk = apply_rope(k, c[: k.shape[2]], s_[: k.shape[2]])
        qq = rq + (rq.detach().to(in_dtype).to(dtype) - rq.detach())
        kk = rk + (rk.detach().to(in_dtype).to(dtype) - rk.detach())
    out = attention(qq, kk, v, dtype=dtype, **kw)
    out.backward(dO.to(dtype))
    return out.detach(), q.grad, k.grad, v.grad


def block_elem_mask(grid: torch.Tensor, block_m: int, block_n: int, N_q: int, N_kv: int) -> torch.Tensor:
    """Element mask (N_q, N_kv) of a boolean block grid (n_q_blocks, n_kv_blocks)."""
    return grid.repeat_interleave(block_m, 0).repeat_interleave(block_n, 1)[:N_q, :N_kv]


# ----------------------------------------------------------------------------------------
# error metrics (the tolerances of the parity bar are written in the tests)
# ----------------------------------------------------------------------------------------
def max_abs(got: torch.Tensor, want: torch.Tensor) -> float:
    return (got.double() - want.double()).abs().max().item() if got.numel() else 0.0


def rel_fro(got: torch.Tensor, want: torch.Tensor) -> float:
    d = (got.double() - want.double()).norm().item()
    n = want.double().norm().item()
    return d / n if n > 0 else d


# ----------------------------------------------------------------------------------------
# seeded inputs (drawn on a CPU generator so the oracle and the kernels see the same bits)
# ----------------------------------------------------------------------------------------
def randn(seed: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)
