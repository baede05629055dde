"""Block-sparse forward / backward parity, shared and per-head masks, both kernel families."""
import numpy as np
import pytest
import torch

import attentionfuse_b200 as af
from oracle import attention_oracle as orc
from tests._util import assert_close, golden, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"


@af.attention
def bs_attn(Q, K, V):
    return af.softmax(af.block_sparse(af.scaled_dot_product(Q, K))) @ V


def make_bs_alibi(h):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.block_sparse(af.alibi(af.scaled_dot_product(Q, K), h))) @ V
    return fn


def bigbird_grid(nq, nk, seed):
    """2 global key blocks, 2 global query block-rows, band of +-1, 3 random extra blocks per row."""
    rng = np.random.default_rng(seed)
    g = np.zeros((nq, nk), dtype=bool)
    g[:, :2] = True
    g[:2, :] = True
    for i in range(nq):
        g[i, max(0, i - 1):min(nk, i + 2)] = True
        free = np.flatnonzero(~g[i])
        if len(free):
            g[i, rng.choice(free, size=min(3, len(free)), replace=False)] = True
    return torch.from_numpy(g)


@pytest.mark.parametrize("block", [64, 128])
@pytest.mark.parametrize("pattern", ["all", "local", "bigbird", "strided"])
def test_shared_mask_forward(block, pattern):
    B, H, N, D = 2, 4, 512, 64
    preds = {
        "all": lambda q, k: torch.ones_like(q, dtype=torch.bool),
        "local": lambda q, k: ((q // block) - (k // block)).abs() <= 1,
        "bigbird": lambda q, k: ((q // block) == 0) | ((k // block) == 0) | (((q // block) - (k // block)).abs() <= 1),
        "strided": lambda q, k: ((q // block) + (k // block)) % 2 == 0,
    }
    bm = af.create_block_mask(preds[pattern], N, N, block, block, device=DEV)
    nb = N // block
    expect = {"all": nb * nb, "local": 3 * nb - 2, "strided": (nb * nb) // 2 + nb % 2}.get(pattern)
    if expect is not None:
        assert bm.n_active == expect
    Q, K, V = qkv(1300, B, H, H, N, N, D, torch.float16)
    qi = torch.arange(N)[:, None].expand(N, N); kj = torch.arange(N)[None, :].expand(N, N)
    want = orc.attention(Q, K, V, elem_mask=preds[pattern](qi, kj))
    got = bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=bm)
    assert_close(got, want, torch.float16, what=f"{pattern} block={block}")


def test_reference_builder_lists():
    """create_block_mask reproduces the lists the reference builder emits (incl. round-up of partial tiles)."""
    g = golden("block_sparse_small_f32")
    preds = {
        "bigbird": (lambda q, k: ((q // 64) == 0) | ((k // 64) == 0) | (((q // 64) - (k // 64)).abs() <= 1), 256),
        "strided": (lambda q, k: ((q // 64) + (k // 64)) % 2 == 0, 256),
        "ragged": (lambda q, k: (q - k).abs() <= 70, 200),
    }
    for name, (fn, n) in preds.items():
        bm = af.create_block_mask(fn, n, n, 64, 64, device="cpu")
        assert bm.n_active == int(g[f"{name}_n_active"])
        assert torch.equal(bm.full_kv_num, g[f"{name}_full_kv_num"])
        assert torch.equal(bm.q_num_blocks, g[f"{name}_q_num_blocks"])
        w = g[f"{name}_full_kv_idx"].shape[1]
        assert torch.equal(bm.full_kv_idx[:, :w], g[f"{name}_full_kv_idx"])
        w = g[f"{name}_q_indices"].shape[1]
        assert torch.equal(bm.q_indices[:, :w], g[f"{name}_q_indices"])
    bm = af.create_block_mask(preds["bigbird"][0], 256, 256, 64, 64, device=DEV)
    got = bs_attn(g["Q"].to(DEV), g["K"].to(DEV), g["V"].to(DEV), block_mask=bm)
    assert_close(got, g["out_bigbird"], torch.float32, what="golden bigbird fp32")


@pytest.mark.parametrize("block,dtype", [(128, torch.float16), (64, torch.bfloat16), (128, torch.float32)])
def test_per_head_masks_forward_backward(block, dtype):
    B, H, N, D = 1, 4, 1024, 64
    nb = N // block
    grids = torch.stack([bigbird_grid(nb, nb, 5000 + h) for h in range(H)])
    bm = af.create_block_mask_per_head(grids, block, block, device=DEV)
    assert bm.per_head and torch.equal(bm.dense_grid(), grids)
    Q, K, V = qkv(1400, B, H, H, N, N, D, dtype)
    dO = orc.randn(1403, (B, H, N, D), dtype)
    want_parts = [orc.attention_grads(Q[:, h:h + 1], K[:, h:h + 1], V[:, h:h + 1], dO[:, h:h + 1],
                                      elem_mask=orc.block_elem_mask(grids[h], block, block, N, N)) for h in range(H)]
    O, dQ, dK, dV = (torch.cat([p[i] for p in want_parts], dim=1) for i in range(4))
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (Q, K, V))
    out = bs_attn(q, k, v, block_mask=bm)
    out.backward(dO.to(DEV))
    assert_close(out, O, dtype, what="per-head O")
    assert_close(q.grad, dQ, dtype, grad=True, what="per-head dQ")
    assert_close(k.grad, dK, dtype, grad=True, what="per-head dK")
    assert_close(v.grad, dV, dtype, grad=True, what="per-head dV")


def test_empty_rows_alibi_gqa_and_errors():
    B, Hq, Hkv, N, D, block = 1, 4, 2, 384, 64, 128
    grid = torch.tensor([[1, 0, 0], [0, 0, 0], [1, 1, 1]], dtype=torch.bool)   # query block 1 sees nothing
    bm = af.BlockMask.from_dense(grid, block, block, device=DEV)
    Q, K, V = qkv(1500, B, Hq, Hkv, N, N, D, torch.bfloat16)
    got = bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=bm)
    want = orc.attention(Q, K, V, elem_mask=orc.block_elem_mask(grid, block, block, N, N))
    assert torch.all(got[:, :, 128:256] == 0) and torch.all(want[:, :, 128:256] == 0)
    assert_close(got, want, torch.bfloat16, what="empty rows")
    from attentionfuse_b200.runtime.dispatch import _alibi_slopes
    got = make_bs_alibi(Hq)(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=bm)
    want = orc.attention(Q, K, V, elem_mask=orc.block_elem_mask(grid, block, block, N, N),
                         slopes=_alibi_slopes(Hq, "cpu", "torch.bfloat16"))
    assert_close(got, want, torch.bfloat16, what="alibi + blocks + gqa")
    with pytest.raises(RuntimeError, match="block_mask"):
        bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV))
    with pytest.raises(TypeError):
        bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=grid)


PREDICATES = {
    # a band that cuts through tiles
    "ragged_band": lambda q, k: (q - k).abs() <= 70,
    # documents of 100 tokens, causal inside each
    "documents": lambda q, k: ((q // 100) == (k // 100)) & (k <= q),
    # a few global keys plus a narrow causal window
    "global_plus_window": lambda q, k: (k < 5) | ((q - k >= 0) & (q - k < 37)),
}


def expected_grads(Q, K, V, dO, elem):
    return orc.attention_grads(Q, K, V, dO, elem_mask=elem)


@pytest.mark.parametrize("pattern", list(PREDICATES))
@pytest.mark.parametrize("case", [(1, 4, 2, 200, 64, 64, torch.bfloat16), (2, 4, 4, 333, 128, 64, torch.float16),
                                  (1, 2, 1, 1000, 128, 128, torch.bfloat16), (1, 2, 2, 200, 64, 64, torch.float32),
                                  (1, 4, 2, 300, 32, 48, torch.bfloat16)],
                         ids=lambda c: f"B{c[0]}H{c[1]}q{c[2]}kv-N{c[3]}-D{c[4]}-blk{c[5]}-{str(c[6]).split('.')[-1]}")
def test_element_exact_partial_tiles(pattern, case):
    """create_block_mask(exact=True): tiles the predicate covers only partly keep exactly its
    elements (a bit matrix per tile) instead of being rounded up as the reference does
    (attnfuse/runtime/block_mask.py:143-154).  Forward and gradients against the oracle fed the
    predicate's own element mask; f16/bf16 with head dim 64/128 on the tensor-core kernels
    (including the single-pass backward at 128), the rest on the exact kernels."""
    B, Hq, Hkv, N, D, block, dtype = case
    fn = PREDICATES[pattern]
    bm = af.create_block_mask(fn, N, N, block, block, device=DEV, exact=True)
    qi = torch.arange(N)[:, None].expand(N, N); kj = torch.arange(N)[None, :].expand(N, N)
    elem = fn(qi, kj)
    assert bm.exact and bm.n_full < bm.n_active
    rounded = af.create_block_mask(fn, N, N, block, block, device=DEV)
    assert rounded.n_active == bm.n_active and not rounded.exact
    Q, K, V = qkv(1600, B, Hq, Hkv, N, N, D, dtype)
    dO = orc.randn(1603, (B, Hq, N, D), dtype)
    O, dQ, dK, dV = expected_grads(Q, K, V, dO, elem)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (Q, K, V))
    out = bs_attn(q, k, v, block_mask=bm)
    out.backward(dO.to(DEV))
    assert_close(out, O, dtype, what=f"exact {pattern} O")
    assert_close(q.grad, dQ, dtype, grad=True, what=f"exact {pattern} dQ")
    assert_close(k.grad, dK, dtype, grad=True, what=f"exact {pattern} dK")
    assert_close(v.grad, dV, dtype, grad=True, what=f"exact {pattern} dV")
    # the rounded-up mask is a different function: it must differ where tiles are partial
    with torch.no_grad():
        up = bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=rounded)
    assert orc.rel_fro(up.float().cpu(), O) > 1e-2


def test_default_block_size_runs_on_the_tensor_core_kernels():
    """Masks at the reference's default block size (64, attnfuse/runtime/block_mask.py:100-103) are
    handed to the kernels at 128 x 128 granularity with quadrant bit matrices, so f16/bf16 problems
    with head dim 64 / 128 stay on the tcgen05 family, forward and backward."""
    from attentionfuse_b200.runtime import _lib
    from attentionfuse_b200.runtime.dispatch import fill_problem
    B, H, N, D, dtype = 1, 4, 1024, 64, torch.float16
    grid = bigbird_grid(N // 64, N // 64, 321)
    bm = af.BlockMask.from_dense(grid, 64, 64, device=DEV)
    assert bm.kernel_lists.block_m == 128 and bm.kernel_lists.kv_slot is not None
    Q, K, V = qkv(1650, B, H, H, N, N, D, dtype)
    dO = orc.randn(1653, (B, H, N, D), dtype)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (Q, K, V))
    for backward in (0, 1):
        p = _lib.AfProblem()
        fill_problem(p, q, k, v, sm_scale=D ** -0.5, mask_kind=_lib.AF_MASK_BLOCKS)
        bm.fill(p, H, backward=bool(backward))
        assert _lib.load().af_query_family(p, backward) == _lib.AF_FAMILY_TCGEN05
    out = bs_attn(q, k, v, block_mask=bm)
    out.backward(dO.to(DEV))
    O, dQ, dK, dV = expected_grads(Q, K, V, dO, orc.block_elem_mask(grid, 64, 64, N, N))
    assert_close(out, O, dtype, what="block 64 O")
    assert_close(q.grad, dQ, dtype, grad=True, what="block 64 dQ")
    assert_close(k.grad, dK, dtype, grad=True, what="block 64 dK")
    assert_close(v.grad, dV, dtype, grad=True, what="block 64 dV")


def test_exact_masks_per_head():
    H, N, D, dtype = 3, 300, 128, torch.bfloat16
    qi = torch.arange(N)[:, None].expand(N, N); kj = torch.arange(N)[None, :].expand(N, N)
    elems = torch.stack([(qi - kj).abs() <= 20 * (h + 1) for h in range(H)])
    bm = af.BlockMask.from_elements(elems, 64, 64, device=DEV)
    assert bm.per_head and bm.exact
    Q, K, V = qkv(1700, 1, H, H, N, N, D, dtype)
    got = bs_attn(Q.to(DEV), K.to(DEV), V.to(DEV), block_mask=bm)
    want = torch.cat([orc.attention(Q[:, h:h + 1], K[:, h:h + 1], V[:, h:h + 1], elem_mask=elems[h]) for h in range(H)], dim=1)
    assert_close(got, want, dtype, what="per-head exact masks")
