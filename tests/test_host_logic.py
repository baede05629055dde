"""Host-side logic that needs no GPU: block-mask builder, work partitioning, the KV-sharded
decode plan (including a world-size-2 gloo run with the CPU oracle standing in for the kernels)."""
import math
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import attentionfuse_b200 as af
from attentionfuse_b200.runtime import partition
from attentionfuse_b200.runtime.sharded_decode import (shard_bounds, local_lengths, sharded_decode, check_gathered,
                                                       cyclic_local_lengths, cyclic_slice)
from oracle import attention_oracle as orc
from tests._util import golden


def test_block_mask_builder_matches_reference_lists():
    g = golden("block_sparse_small_f32")
    preds = {
        "bigbird": (lambda q, k: ((q // 64) == 0) | ((k // 64) == 0) | (((q // 64) - (k // 64)).abs() <= 1), 256),
        "strided": (lambda q, k: ((q // 64) + (k // 64)) % 2 == 0, 256),
        "ragged": (lambda q, k: (q - k).abs() <= 70, 200),     # partial tiles are rounded up
    }
    for name, (fn, n) in preds.items():
        bm = af.create_block_mask(fn, n, n, 64, 64, device="cpu")
        assert bm.n_active == int(g[f"{name}_n_active"]) == bm.n_full
        assert torch.equal(bm.full_kv_num, g[f"{name}_full_kv_num"])
        assert torch.equal(bm.q_num_blocks, g[f"{name}_q_num_blocks"])
        assert int(bm.kv_num_blocks.sum()) == int(g[f"{name}_kv_num_blocks"].sum()) == 0
        for mine, ref in ((bm.full_kv_idx, g[f"{name}_full_kv_idx"]), (bm.q_indices, g[f"{name}_q_indices"])):
            assert torch.equal(mine[:, : ref.shape[1]], ref)


def test_exact_masks_and_the_kernels_tile_view_reproduce_the_elements():
    """The lists a launch sees (128 x 128 tiles, a bit matrix for every partly covered tile, both
    orientations) decode back to exactly the element mask they were built from: an exact band mask
    at block 64 and a block-level mask at block 64 that is re-tiled into quadrant patterns."""
    from attentionfuse_b200.runtime.block_mask import BlockMask

    def decode(kl, n_q, n_k):
        def unpack(words):                       # (rows, W) int64 -> (rows, 64 W) bool
            return ((words.unsqueeze(-1) >> torch.arange(64)) & 1).bool().flatten(-2)
        T = kl.block_m
        by_q = torch.zeros(kl.kv_num.shape[0] * T, kl.q_num.shape[0] * T, dtype=torch.bool)
        by_k = torch.zeros_like(by_q)
        for qb in range(kl.kv_num.shape[0]):
            for e in range(int(kl.kv_num[qb])):
                kb = int(kl.kv_idx[qb, e]); s = -1 if kl.kv_slot is None else int(kl.kv_slot[qb, e])
                by_q[qb * T:(qb + 1) * T, kb * T:(kb + 1) * T] = True if s < 0 else unpack(kl.kv_bits[s])[:, :T]
        for kb in range(kl.q_num.shape[0]):
            for e in range(int(kl.q_num[kb])):
                qb = int(kl.q_idx[kb, e]); s = -1 if kl.q_slot is None else int(kl.q_slot[kb, e])
                by_k[qb * T:(qb + 1) * T, kb * T:(kb + 1) * T] = True if s < 0 else unpack(kl.q_bits[s])[:, :T].T
        return by_q[:n_q, :n_k], by_k[:n_q, :n_k]

    N = 200
    fn = lambda q, k: (q - k).abs() <= 70
    qi = torch.arange(N)[:, None].expand(N, N); kj = torch.arange(N)[None, :].expand(N, N)
    bm = af.create_block_mask(fn, N, N, 64, 64, device="cpu", exact=True)
    assert bm.n_full < bm.n_active
    assert bm.kv_num_blocks.sum() + bm.full_kv_num.sum() == bm.n_active
    a, b = decode(bm.kernel_lists, N, N)
    assert torch.equal(a, fn(qi, kj)) and torch.equal(b, fn(qi, kj))
    grid = torch.rand(7, 5, generator=torch.Generator().manual_seed(3)) > 0.5
    bm = BlockMask.from_dense(grid, 64, 64, device="cpu")
    want = orc.block_elem_mask(grid, 64, 64, 7 * 64, 5 * 64)
    a, b = decode(bm.kernel_lists, 7 * 64, 5 * 64)
    assert bm.kernel_lists.block_m == 128 and torch.equal(a, want) and torch.equal(b, want)
    assert torch.equal(bm.dense_grid(), grid)


def test_block_mask_per_head_roundtrip_and_bigbird_counts():
    rng = np.random.default_rng(0)
    grids = torch.from_numpy(rng.random((3, 7, 5)) < 0.4)
    grids[1, 2] = False                                         # a query block with no active key block
    bm = af.create_block_mask_per_head(grids, 128, 128, device="cpu")
    assert bm.per_head and torch.equal(bm.dense_grid(), grids) and bm.n_active == int(grids.sum())
    assert torch.equal(bm.q_num_blocks, grids.sum(1).to(torch.int32))
    with pytest.raises(ValueError):
        af.create_block_mask_per_head(grids[0], 128, 128, device="cpu")


def test_partition_covers_every_unit_once():
    for B, H, world in ((4, 12, 8), (4, 8, 8), (2, 16, 3), (1, 1, 4), (3, 5, 7)):
        seen = np.zeros((B, H), dtype=int)
        sizes = []
        for r in range(world):
            rects = partition.shard(B, H, world, r)
            assert len(rects) <= 3
            n = 0
            for b0, b1, h0, h1 in rects:
                seen[b0:b1, h0:h1] += 1
                n += (b1 - b0) * (h1 - h0)
            sizes.append(n)
        assert (seen == 1).all() and max(sizes) - min(sizes) <= 1
    Q, K, V = torch.zeros(4, 32, 2, 8), torch.zeros(4, 8, 2, 8), torch.zeros(4, 8, 2, 8)
    q, k, v = partition.slice_qkv(Q, K, V, (1, 2, 2, 6))
    assert q.shape == (1, 16, 2, 8) and k.shape == (1, 4, 2, 8)


def test_shard_plan():
    assert [shard_bounds(32768, 8, r) for r in (0, 7)] == [(0, 4096), (28672, 32768)]
    assert shard_bounds(10, 4, 3) == (9, 10) and shard_bounds(10, 4, 2) == (6, 9)
    lens = torch.tensor([32768, 16384, 20000, 5])
    assert local_lengths(lens, 16384, 20480).tolist() == [4096, 0, 3616, 0]
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def test_cyclic_layout_is_balanced_and_exact():
    lens = torch.tensor([32768, 16384, 20000, 5, 0, 2048 + 17])
    for world in (2, 4, 8):
        per = torch.stack([cyclic_local_lengths(lens, r, world) for r in range(world)]).long()
        assert torch.equal(per.sum(0), lens)
        assert (per.max(0).values - per.min(0).values).max().item() <= 256
    t = torch.arange(2 * 1 * 2048 * 1).view(2, 1, 2048, 1)
    parts = [cyclic_slice(t, r, 4) for r in range(4)]
    assert parts[1][0, 0, :3, 0].tolist() == [256, 257, 258] and parts[1][0, 0, 256, 0].item() == 1024 + 256
    # the first n local keys of rank r are exactly its keys below the global length
    L = 1500
    for r in range(4):
        n = int(cyclic_local_lengths(torch.tensor([L]), r, 4))
        assert (parts[r][0, 0, :n, 0] < L).all() and (parts[r][0, 0, n:, 0] >= L).all()
    with pytest.raises(ValueError):
        cyclic_slice(t, 0, 3)


def _cpu_partial(Q, K, V, sm_scale, bias_kind, lens, kv_offset, q_positions, slopes):
    out, lse = orc.attention(Q, K, V, scale=sm_scale, kv_lens=lens.long(), return_lse=True)
    return torch.cat([out[:, :, 0, :], lse], dim=-1).float()


def _cpu_combine(gathered, out):
    lse = gathered[..., -1]
    m = lse.max(dim=0).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(lse - m)
    num = (w.unsqueeze(-1) * torch.nan_to_num(gathered[..., :-1])).sum(0)
    den = w.sum(0).unsqueeze(-1)
    out.copy_((num / torch.where(den == 0, torch.ones_like(den), den)).unsqueeze(2).to(out.dtype))
    return out


def _worker(rank, world, port, fail_rank, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, L, D = 3, 8, 2, 96, 32
        Q, K, V = (orc.randn(5 + i, (B, h, n, D), torch.float32) for i, (h, n) in enumerate(((Hq, 1), (Hkv, L), (Hkv, L))))
        lens = torch.tensor([96, 40, 49], dtype=torch.int32)
        lo, hi = shard_bounds(L, world, rank)

        def partial_fn(*a):
            p = _cpu_partial(*a)
            if rank == fail_rank:
                p[..., -1] = float("nan")              # a rank that produced garbage
            return p

        gathered = torch.empty(world, B, Hq, D + 1)
        out = sharded_decode(Q, K[:, :, lo:hi], V[:, :, lo:hi], lens, L, rank, world, local_partial=partial_fn,
                             combine=_cpu_combine, gather_buffer=gathered)
        if fail_rank is not None:
            try:
                check_gathered(gathered)
                ret[rank] = "no error raised"
            except RuntimeError as e:
                ret[rank] = str(e)
        else:
            want = orc.attention(Q, K, V, kv_lens=lens.long())
            ret[rank] = (out - want).abs().max().item()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [None, 1])
def test_sharded_decode_world2_gloo(fail_rank):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29500 + (os.getpid() % 2000) + (0 if fail_rank is None else 1)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_rank, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    if fail_rank is None:
        assert all(v < 1e-5 for v in ret.values()), dict(ret)
    else:
        assert all("NaN log-sum-exp" in v and "[1]" in v for v in ret.values()), dict(ret)


def test_hf_hook_hands_padded_batches_and_unaligned_causal_to_sdpa(monkeypatch):
    """Masks the kernel's plain causal rule cannot express go to the SDPA backend untouched: a
    left-padded batch (whole key columns masked for one row of the batch) and causal attention
    over a rectangular score matrix without a mask.  The fall-back is decided on the host, so no
    GPU is involved."""
    pytest.importorskip("transformers")
    import attentionfuse_b200.integrations.hf as hf
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    calls = []

    def fake_sdpa(module, q, k, v, mask, **kw):
        calls.append(kw.get("is_causal"))
        return torch.zeros(q.shape[0], q.shape[2], q.shape[1], q.shape[3]), None
    monkeypatch.setitem(ALL_ATTENTION_FUNCTIONS, "sdpa", fake_sdpa)
    B, H, N, D = 2, 2, 8, 16
    q = k = v = torch.zeros(B, H, N, D)
    neg = torch.finfo(torch.float32).min
    mask = torch.triu(torch.full((N, N), neg), diagonal=1).expand(B, 1, N, N).clone()
    assert hf._every_key_visible_to_last_row(mask) and hf._is_pure_causal_mask(mask, N, N)
    mask[1, :, :, :3] = neg                               # row 1 of the batch is left-padded by 3
    assert hf._is_pure_causal_mask(mask, N, N)            # the corner probe alone is fooled
    hf.attnfuse_attention_forward(torch.nn.Identity(), q, k, v, mask)
    assert len(calls) == 1
    step_mask = torch.zeros(B, 1, 1, N)
    step_mask[1, :, :, :3] = neg                          # the same padding during a decode step
    hf.attnfuse_attention_forward(torch.nn.Identity(), q[:, :, :1], k, v, step_mask)
    assert len(calls) == 2
    hf.attnfuse_attention_forward(torch.nn.Identity(), q[:, :, :4], k, v, None, is_causal=True)
    assert len(calls) == 3 and calls[2] is True
