"""Decode (query length 1) parity: split-K kernel + combine against the oracle, with
per-sequence lengths, ALiBi, GQA / MQA geometries and the KV-sharded merge."""
import pytest
import torch

import attentionfuse_b200 as af
from attentionfuse_b200.runtime.dispatch import _alibi_slopes
from attentionfuse_b200.runtime.flash_decode import run_flash_decode, combine_gathered
from attentionfuse_b200.runtime.sharded_decode import (shard_bounds, sharded_decode, ShardedDecodePlan, PeerExchange,
                                                       cyclic_slice, cyclic_local_lengths)
from oracle import attention_oracle as orc
from tests._util import assert_close, golden, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"


@af.attention
def dense(Q, K, V):
    return af.softmax(af.scaled_dot_product(Q, K)) @ V


def make_alibi(h):
    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.alibi(af.scaled_dot_product(Q, K), h)) @ V
    return fn


def lens_for(seed, B, L):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(L // 2, L + 1, (B,), generator=g, dtype=torch.int32)


GEOM = [(32, 8), (64, 8), (64, 1), (8, 8), (12, 4)]


@pytest.mark.parametrize("heads", GEOM, ids=lambda h: f"{h[0]}q{h[1]}kv")
@pytest.mark.parametrize("L", [256, 1000, 4096])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_ragged(heads, L, dtype):
    Hq, Hkv = heads
    B, D = 3, 128
    Q, K, V = qkv(900 + L, B, Hq, Hkv, 1, L, D, dtype)
    lens = lens_for(L, B, L)
    got = dense(Q.to(DEV), K.to(DEV), V.to(DEV), kv_lens=lens.to(DEV))
    want = orc.attention(Q, K, V, kv_lens=lens)
    assert_close(got, want, dtype, what=f"decode {heads} L={L}")
    got_full = dense(Q.to(DEV), K.to(DEV), V.to(DEV))
    assert_close(got_full, orc.attention(Q, K, V), dtype, what=f"decode full {heads} L={L}")


def test_decode_d64_and_alibi():
    B, Hq, Hkv, L, D = 2, 8, 2, 777, 64
    Q, K, V = qkv(950, B, Hq, Hkv, 1, L, D, torch.float16)
    lens = lens_for(5, B, L)
    assert_close(dense(Q.to(DEV), K.to(DEV), V.to(DEV), kv_lens=lens.to(DEV)),
                 orc.attention(Q, K, V, kv_lens=lens), torch.float16, what="d64")
    slopes = _alibi_slopes(Hq, "cpu", "float16")
    got = make_alibi(Hq)(Q.to(DEV), K.to(DEV), V.to(DEV))
    assert_close(got, orc.attention(Q, K, V, slopes=slopes), torch.float16, what="alibi decode")
    got = make_alibi(Hq)(Q.to(DEV), K.to(DEV), V.to(DEV), kv_lens=lens.to(DEV))
    assert_close(got, orc.attention(Q, K, V, slopes=slopes, kv_lens=lens), torch.float16, what="alibi ragged")


def test_decode_golden_and_fp32_route():
    g = golden("decode_small_f32")
    # fp32 takes the general forward kernel (the decode kernels are half precision)
    got = dense(g["Q"].to(DEV), g["K"].to(DEV), g["V"].to(DEV))
    assert_close(got, g["full"], torch.float32, what="fp32 decode via forward kernel")
    Q, K, V = (g[k].to(torch.bfloat16) for k in ("Q", "K", "V"))
    got = dense(Q.to(DEV), K.to(DEV), V.to(DEV), kv_lens=g["kv_lens"].to(DEV))
    assert_close(got, orc.attention(Q, K, V, kv_lens=g["kv_lens"]), torch.bfloat16, what="golden ragged bf16")


@pytest.mark.parametrize("heads", [(3, 1), (5, 5), (9, 3), (1, 1)], ids=lambda h: f"{h[0]}q{h[1]}kv")
@pytest.mark.parametrize("splits", [1, 3, 5])
@pytest.mark.parametrize("B", [1, 3])
def test_odd_partial_row_counts(heads, splits, B):
    """num_splits * B * H_q odd: the (m, l, acc) partials are carved from one allocation, and acc
    must start on a 16-byte boundary whatever the row count."""
    Hq, Hkv = heads
    L, D = 1536, 128
    Q, K, V = qkv(990 + Hq, B, Hq, Hkv, 1, L, D, torch.bfloat16)
    lens = lens_for(17 + B, B, L)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    out = torch.full_like(q, float("nan"))
    run_flash_decode(None, q, k, v, 1.0 / D ** 0.5, 0, Hkv, out, kv_lens=lens.to(DEV), num_splits=splits)
    assert_close(out, orc.attention(Q, K, V, kv_lens=lens), torch.bfloat16, what=f"odd rows {heads} S={splits} B={B}")
    if splits == 3:   # the split count the heuristic picks at this length goes the same way
        assert_close(dense(q, k, v), orc.attention(Q, K, V), torch.bfloat16, what=f"odd rows auto {heads} B={B}")


def build_graph(variant, H, W):
    @af.attention
    def fn(Q, K, V):
        s = af.rope(Q, K) if "rope" in variant else af.scaled_dot_product(Q, K)
        if "alibi" in variant:
            s = af.alibi(s, H)
        if "causal" in variant:
            s = af.causal(s)
        if "window" in variant:
            s = af.sliding_window(s, W)
        return af.softmax(s) @ V
    return fn


@pytest.mark.parametrize("variant", ["causal", "window", "causal_alibi", "causal_rope", "causal_rope_alibi", "window_rope"])
@pytest.mark.parametrize("geom", [(32, 8, 128), (64, 1, 128), (8, 2, 64)], ids=lambda g: f"{g[0]}q{g[1]}kv_d{g[2]}")
def test_single_row_with_masks_and_rotation_runs_split_k(variant, geom):
    """One query row at position p of a longer cache with a causal or window mask, ALiBi measured
    from p and RoPE: served by the split-K decode kernels (two launches, K/V read once per KV head),
    not by a 128-row forward tile.  The reference's decode path refuses all of these
    (attnfuse/runtime/flash_decode.py:46-65)."""
    Hq, Hkv, D = geom
    B, L, W, dtype = 2, 3000, 700, torch.bfloat16
    p = 2345                                            # keys past p exist in the cache and must not be seen
    Q, K, V = qkv(1700 + Hq, B, Hq, Hkv, 1, L, D, dtype)
    kw, okw = {}, {"q_offset": p}
    if "rope" in variant:
        cos, sin = orc.build_rope_cache(L, D, 500000.0, dtype)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV)); okw.update(cos=cos, sin=sin)
    if "alibi" in variant:
        okw.update(slopes=_alibi_slopes(Hq, "cpu", str(dtype)), q_positions=torch.full((B,), p))
    okw["causal"] = "causal" in variant
    if "window" in variant:
        okw["window"] = W
    want = orc.attention(Q, K, V, **okw)
    from attentionfuse_b200.runtime import _lib
    before = _lib.launch_count()
    got = build_graph(variant, Hq, W)(Q.to(DEV), K.to(DEV), V.to(DEV), q_offset=p, **kw)
    assert _lib.launch_count() - before == 2, "expected the split-K pair of launches"
    assert_close(got, want, dtype, what=f"single row {variant} {geom}")


def test_ragged_batch_decodes_with_rotation_at_each_sequence_end():
    """Per-sequence lengths and per-sequence query positions (the new token is the last valid key
    of its sequence): causal + RoPE through the split-K kernels, one oracle call per batch row."""
    B, Hq, Hkv, L, D, dtype = 4, 16, 4, 2048, 128, torch.float16
    Q, K, V = qkv(1800, B, Hq, Hkv, 1, L, D, dtype)
    lens = lens_for(77, B, L)
    cos, sin = orc.build_rope_cache(L, D, 10000.0, dtype)

    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.causal(af.rope(Q, K))) @ V

    got = fn(Q.to(DEV), K.to(DEV), V.to(DEV), cos=cos.to(DEV), sin=sin.to(DEV), kv_lens=lens.to(DEV),
             q_offset=(lens - 1).to(DEV))
    for b in range(B):
        n = int(lens[b])
        want = orc.attention(Q[b:b + 1], K[b:b + 1, :, :n], V[b:b + 1, :, :n], causal=True, cos=cos, sin=sin, q_offset=n - 1)
        assert_close(got[b:b + 1], want, dtype, what=f"ragged rope row {b}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cache_of_rotated_keys_rotates_the_query_row_only(dtype):
    """A serving cache holds keys that were rotated when they were written: `kv_rotated=True`
    rotates the query row alone, at its position.  Same result as rotating the stored keys on
    load (both round the rotated key to the cache type once), and the oracle's."""
    from attentionfuse_b200.rope_utils import apply_rope
    B, Hq, Hkv, L, D = 3, 16, 4, 3000, 128
    Q, K, V = qkv(1850, B, Hq, Hkv, 1, L, D, dtype)
    lens = lens_for(79, B, L)
    cos, sin = orc.build_rope_cache(L, D, 500000.0, dtype)

    @af.attention
    def fn(Q, K, V):
        return af.softmax(af.causal(af.rope(Q, K))) @ V

    kw = dict(cos=cos.to(DEV), sin=sin.to(DEV), kv_lens=lens.to(DEV), q_offset=(lens - 1).to(DEV))
    on_load = fn(Q.to(DEV), K.to(DEV), V.to(DEV), **kw)
    K_rot = apply_rope(K.to(DEV).float(), cos.to(DEV).float(), sin.to(DEV).float()).to(dtype)   # fp32 math, one rounding
    stored = fn(Q.to(DEV), K_rot, V.to(DEV), kv_rotated=True, **kw)
    assert (stored.float() - on_load.float()).abs().max().item() <= 4e-3
    for b in range(B):
        n = int(lens[b])
        want = orc.attention(Q[b:b + 1], K[b:b + 1, :, :n], V[b:b + 1, :, :n], causal=True, cos=cos, sin=sin, q_offset=n - 1)
        assert_close(stored[b:b + 1], want, dtype, what=f"rotated cache row {b}")
    with pytest.raises(ValueError):
        fn(Q.to(DEV).expand(B, Hq, 4, D).contiguous(), K_rot[:, :, :4], V.to(DEV)[:, :, :4], cos=cos.to(DEV), sin=sin.to(DEV), kv_rotated=True)


@pytest.mark.parametrize("splits", [1, 2, 7, 16])
def test_split_counts_agree(splits):
    B, Hq, Hkv, L, D = 2, 32, 8, 2048, 128
    Q, K, V = qkv(970, B, Hq, Hkv, 1, L, D, torch.bfloat16)
    lens = torch.tensor([1500, 64], dtype=torch.int32)
    out = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    run_flash_decode(None, Q.to(DEV), K.to(DEV), V.to(DEV), 1.0 / D ** 0.5, 0, Hkv, out,
                     kv_lens=lens.to(DEV), num_splits=splits)
    assert_close(out, orc.attention(Q, K, V, kv_lens=lens), torch.bfloat16, what=f"splits={splits}")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_kv_sharded_merge_emulated(world):
    """The multi-GPU path on one GPU: every rank's local decode runs as its own pair of launches
    (nothing waits on another rank), the partials are stacked as an all-gather would place them,
    and the gathered-combine kernel merges them."""
    B, Hq, Hkv, L, D = 4, 32, 8, 4096, 128
    Q, K, V = qkv(990, B, Hq, Hkv, 1, L, D, torch.bfloat16)
    lens = torch.tensor([4096, 2048, 2049, 517], dtype=torch.int32)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    gathered = torch.empty(world, B, Hq, D + 1, dtype=torch.float32, device=DEV)
    for r in range(world):
        lo, hi = shard_bounds(L, world, r)

        def fake_gather(buf, partial, r=r):
            gathered[r].copy_(partial)
        sharded_decode(q, k[:, :, lo:hi], v[:, :, lo:hi], lens.to(DEV), L, r, world,
                       all_gather=fake_gather, combine=lambda buf, out: None)
    out = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    combine_gathered(gathered, out)
    assert_close(out, orc.attention(Q, K, V, kv_lens=lens), torch.bfloat16, what=f"sharded world={world}")
    # rank with no valid keys for a row must report LSE = -inf there
    assert torch.isinf(gathered[world - 1, 3, :, D]).all()


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("layout", ["contiguous", "cyclic"])
def test_sharded_plan_layouts_emulated(world, layout):
    """ShardedDecodePlan on one GPU: each rank's plan runs its local launches, the partials are
    stacked by hand in place of the all-gather, the merge kernel produces the unsharded result."""
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    B, Hq, Hkv, L, D = 4, 32, 8, 4096, 128
    Q, K, V = qkv(995, B, Hq, Hkv, 1, L, D, torch.bfloat16)
    lens = torch.tensor([4096, 2048, 2049, 300], dtype=torch.int32)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    gathered = torch.empty(world, B, Hq, D + 1, dtype=torch.float32, device=DEV)
    total_local = torch.zeros(B, dtype=torch.int64)
    for r in range(world):
        plan = ShardedDecodePlan(B, Hq, Hkv, D, L, r, world, lens, torch.device(DEV, 0), torch.bfloat16, layout=layout)
        if layout == "cyclic":
            kl, vl = cyclic_slice(k, r, world).contiguous(), cyclic_slice(v, r, world).contiguous()
        else:
            kl, vl = k[:, :, plan.lo:plan.hi], v[:, :, plan.lo:plan.hi]
        rfd(None, q, kl, vl, plan.sm_scale, 0, Hkv, None, kv_lens=plan.lens_local, kv_offset=plan.kv_offset,
            partial=plan.partial, num_splits=plan.num_splits, workspace=plan.workspace)
        gathered[r].copy_(plan.partial)
        total_local += plan.lens_local.cpu().long()
    assert torch.equal(total_local, lens.long())               # every valid key is owned exactly once
    out = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    combine_gathered(gathered, out)
    assert_close(out, orc.attention(Q, K, V, kv_lens=lens), torch.bfloat16, what=f"{layout} world={world}")
    if layout == "cyclic":
        per_rank = torch.stack([cyclic_local_lengths(lens, r, world) for r in range(world)]).long()
        assert (per_rank.max(0).values - per_rank.min(0).values).max().item() <= 256   # balanced to one block


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("layout", ["contiguous", "cyclic"])
def test_sharded_plan_with_alibi_sees_true_key_positions(world, layout):
    """ALiBi measures the distance of every key from the query row on the true key axis: a rank of
    the block-cyclic layout passes its rank offset and the block / stride of the dealing
    (AfDecodeParams.kv_pos_block / kv_pos_stride), a contiguous shard its first position."""
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    B, Hq, Hkv, L, D = 3, 16, 4, 4096, 128
    Q, K, V = qkv(1995, B, Hq, Hkv, 1, L, D, torch.bfloat16)
    lens = torch.tensor([4096, 2049, 700], dtype=torch.int32)
    slopes = _alibi_slopes(Hq, "cpu", "torch.bfloat16")
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    gathered = torch.empty(world, B, Hq, D + 1, dtype=torch.float32, device=DEV)
    for r in range(world):
        plan = ShardedDecodePlan(B, Hq, Hkv, D, L, r, world, lens, torch.device(DEV, 0), torch.bfloat16, layout=layout,
                                 bias_kind=1, slopes=slopes)
        if layout == "cyclic":
            kl, vl = cyclic_slice(k, r, world).contiguous(), cyclic_slice(v, r, world).contiguous()
        else:
            kl, vl = k[:, :, plan.lo:plan.hi], v[:, :, plan.lo:plan.hi]
        rfd(None, q, kl, vl, plan.sm_scale, 1, Hkv, None, kv_lens=plan.lens_local, alibi_slopes=plan.slopes,
            kv_offset=plan.kv_offset, q_positions=plan.q_positions, partial=plan.partial, num_splits=plan.num_splits,
            workspace=plan.workspace, **plan.kv_pos)
        gathered[r].copy_(plan.partial)
    out = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    combine_gathered(gathered, out)
    assert_close(out, orc.attention(Q, K, V, kv_lens=lens, slopes=slopes), torch.bfloat16, what=f"alibi {layout} world={world}")


def _emulated_exchanges(world, B, Hq, D, wait_cycles=0):
    from attentionfuse_b200.runtime import _lib
    n = int(_lib.load().af_decode_exchange_bytes(world, B, Hq, D)) // 4
    bufs = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(world)]
    return [PeerExchange(world, r, B, Hq, D, torch.device(DEV, 0), peer_buffers=bufs, wait_cycles=wait_cycles)
            for r in range(world)]


@pytest.mark.parametrize("world", [2, 8])
def test_peer_exchange_kernels_emulated(world):
    """The fused exchange on one GPU: the "ranks" share the device, their buffers stand in for
    symmetric memory, and launches are strictly sequential (all pushes of a step, then the merges),
    so no kernel ever waits for a later launch.  Three steps exercise both buffer parities."""
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    B, Hq, Hkv, L, D = 4, 32, 8, 4096, 128
    ex = _emulated_exchanges(world, B, Hq, D)
    for step in range(3):
        Q, K, V = qkv(2000 + step, B, Hq, Hkv, 1, L, D, torch.bfloat16)
        lens = torch.tensor([4096, 2048 + step, 2049, 300], dtype=torch.int32)
        q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
        plans = [ShardedDecodePlan(B, Hq, Hkv, D, L, r, world, lens, torch.device(DEV, 0), torch.bfloat16, layout="cyclic")
                 for r in range(world)]
        for r, plan in enumerate(plans):
            rfd(None, q, cyclic_slice(k, r, world).contiguous(), cyclic_slice(v, r, world).contiguous(), plan.sm_scale,
                0, Hkv, None, kv_lens=plan.lens_local, num_splits=plan.num_splits, workspace=plan.workspace,
                exchange=ex[r])
        want = orc.attention(Q, K, V, kv_lens=lens)
        for r in range(world):
            out = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
            ex[r].wait_merge(out)
            ex[r].check_status()
            assert_close(out, want, torch.bfloat16, what=f"p2p exchange world={world} rank={r} step={step}")


@pytest.mark.parametrize("ctas", [1, 7, 100, 296, 1000])
@pytest.mark.parametrize("geom", [(32, 8, 128), (64, 1, 128), (9, 3, 128), (8, 2, 64), (80, 1, 64)],
                         ids=lambda g: f"{g[0]}q{g[1]}kv_d{g[2]}")
def test_balanced_schedule(ctas, geom):
    """balanced_ctas: every CTA takes an equal share of the 64-key tiles of all sequences laid end to
    end, so a share may end inside one (batch, kv head) unit and start the next.  Ragged lengths
    (one sequence empty, one of a single key), CTA counts below and far above the tile count."""
    Hq, Hkv, D = geom
    B, L, dtype = 5, 2500, torch.bfloat16
    Q, K, V = qkv(2600 + Hq, B, Hq, Hkv, 1, L, D, dtype)
    lens = torch.tensor([2500, 1, 1300, 0, 777], dtype=torch.int32)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    k[3] = float("nan"); v[3] = float("nan")          # the empty sequence's cache must not be read into the result
    out = torch.full_like(q, float("nan"))
    run_flash_decode(None, q, k, v, 1.0 / D ** 0.5, 0, Hkv, out, kv_lens=lens.to(DEV), balanced_ctas=ctas)
    want = orc.attention(Q, K, V, kv_lens=lens)
    assert_close(out, want, dtype, what=f"balanced {geom} ctas={ctas}")


@pytest.mark.parametrize("variant", ["causal_alibi", "window_rope"])
def test_balanced_schedule_with_masks_and_rotation(variant):
    Hq, Hkv, D, B, L, W, dtype = 16, 4, 128, 3, 3000, 700, torch.bfloat16
    p = 2345
    Q, K, V = qkv(2700, B, Hq, Hkv, 1, L, D, dtype)
    kw, okw = {}, {"q_offset": p, "causal": "causal" in variant}
    if "rope" in variant:
        cos, sin = orc.build_rope_cache(L, D, 500000.0, dtype)
        kw.update(cos=cos.to(DEV), sin=sin.to(DEV)); okw.update(cos=cos, sin=sin)
    slopes = None
    if "alibi" in variant:
        slopes = _alibi_slopes(Hq, "cpu", str(dtype))
        okw.update(slopes=slopes, q_positions=torch.full((B,), p))
    if "window" in variant:
        okw["window"] = W
    out = torch.empty(B, Hq, 1, D, dtype=dtype, device=DEV)
    run_flash_decode(None, Q.to(DEV), K.to(DEV), V.to(DEV), 1.0 / D ** 0.5, 1 if slopes is not None else 0, Hkv, out,
                     alibi_slopes=slopes, q_position=p, mask_kind=1 if "causal" in variant else 2, window=W,
                     balanced_ctas=148, **kw)
    assert_close(out, orc.attention(Q, K, V, **okw), dtype, what=f"balanced {variant}")


@pytest.mark.parametrize("balanced", [False, True], ids=["split_grid", "balanced"])
@pytest.mark.parametrize("world", [1, 2, 8])
def test_single_launch_sharded_step_emulated(world, balanced):
    """The KV-sharded step as one kernel (split-K, per-unit merge + push, wait, final merge).  With
    one rank the whole step is a single launch on this GPU.  With more "ranks" than GPUs the launch
    is issued in its two halves -- every rank's push half first, then every rank's merge half -- so
    that no kernel waits for a later launch; the code of both halves is the code of the whole."""
    from attentionfuse_b200.runtime import _lib
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    B, Hq, Hkv, L, D = 4, 32, 8, 4096, 128
    ex = _emulated_exchanges(world, B, Hq, D)
    for step in range(3):
        Q, K, V = qkv(2300 + step, B, Hq, Hkv, 1, L, D, torch.bfloat16)
        lens = torch.tensor([4096, 2048 + step, 2049, 300], dtype=torch.int32)
        q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
        want = orc.attention(Q, K, V, kv_lens=lens)
        plans = [ShardedDecodePlan(B, Hq, Hkv, D, L, r, world, lens, torch.device(DEV, 0), torch.bfloat16, layout="cyclic",
                                   exchange="fused", peer_exchange=ex[r], balanced=balanced) for r in range(world)]
        outs = [torch.full((B, Hq, 1, D), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
        kl = [cyclic_slice(k, r, world).contiguous() for r in range(world)]
        vl = [cyclic_slice(v, r, world).contiguous() for r in range(world)]
        before = _lib.launch_count()
        for mode in ((3,) if world == 1 else (1, 2)):
            for r, plan in enumerate(plans):
                rfd(None, q, kl[r], vl[r], plan.sm_scale, 0, Hkv, outs[r], kv_lens=plan.lens_local,
                    num_splits=plan.num_splits, workspace=plan.workspace, exchange=ex[r], exchange_mode=mode,
                    balanced_ctas=plan.balanced_ctas)
        if world == 1:
            assert _lib.launch_count() - before == 1
        for r in range(world):
            ex[r].check_status()
            assert_close(outs[r], want, torch.bfloat16, what=f"single-launch step world={world} rank={r} step={step}")


def test_single_launch_step_wait_runs_out_without_hanging():
    """A peer that never pushes: the waiting CTAs give up after the bound, the status word is set,
    nothing hangs, and the device stays usable."""
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    world, B, Hq, Hkv, L, D = 2, 2, 8, 2, 1024, 64
    ex = _emulated_exchanges(world, B, Hq, D, wait_cycles=2_000_000)      # ~1 ms
    Q, K, V = qkv(2400, B, Hq, Hkv, 1, L, D, torch.float16)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    plan = ShardedDecodePlan(B, Hq, Hkv, D, L, 0, world, None, torch.device(DEV, 0), torch.float16, layout="cyclic",
                             exchange="fused", peer_exchange=ex[0])
    out = torch.zeros(B, Hq, 1, D, dtype=torch.float16, device=DEV)
    rfd(None, q, cyclic_slice(k, 0, world).contiguous(), cyclic_slice(v, 0, world).contiguous(), plan.sm_scale, 0, Hkv,
        out, kv_lens=plan.lens_local, num_splits=plan.num_splits, workspace=plan.workspace, exchange=ex[0], exchange_mode=3)
    with pytest.raises(RuntimeError, match="did not arrive"):
        ex[0].check_status()
    assert_close(dense(q, k, v), orc.attention(Q, K, V), torch.float16, what="after timeout")


def test_peer_exchange_wait_runs_out_without_hanging():
    """A rank that never pushes: the merge kernel's bounded wait ends, the status word is set, the
    host raises, and the context stays usable.  (The failure is an absent message, not a fault.)"""
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode as rfd
    world, B, Hq, Hkv, L, D = 2, 2, 8, 2, 1024, 64
    ex = _emulated_exchanges(world, B, Hq, D, wait_cycles=2_000_000)      # ~1 ms
    Q, K, V = qkv(2100, B, Hq, Hkv, 1, L, D, torch.float16)
    q, k, v = Q.to(DEV), K.to(DEV), V.to(DEV)
    plan = ShardedDecodePlan(B, Hq, Hkv, D, L, 0, world, None, torch.device(DEV, 0), torch.float16, layout="cyclic")
    rfd(None, q, cyclic_slice(k, 0, world).contiguous(), cyclic_slice(v, 0, world).contiguous(), plan.sm_scale, 0, Hkv,
        None, kv_lens=plan.lens_local, num_splits=plan.num_splits, workspace=plan.workspace, exchange=ex[0])
    out = torch.zeros(B, Hq, 1, D, dtype=torch.float16, device=DEV)
    ex[0].wait_merge(out)                    # rank 1 never pushed
    with pytest.raises(RuntimeError, match="did not arrive"):
        ex[0].check_status()
    # the device still works and a complete step succeeds afterwards
    ex2 = _emulated_exchanges(world, B, Hq, D)
    for r in range(world):
        p = ShardedDecodePlan(B, Hq, Hkv, D, L, r, world, None, torch.device(DEV, 0), torch.float16, layout="cyclic")
        rfd(None, q, cyclic_slice(k, r, world).contiguous(), cyclic_slice(v, r, world).contiguous(), p.sm_scale, 0, Hkv,
            None, kv_lens=p.lens_local, num_splits=p.num_splits, workspace=p.workspace, exchange=ex2[r])
    ex2[1].wait_merge(out)
    ex2[1].check_status()
    assert_close(out, orc.attention(Q, K, V), torch.float16, what="after timeout")


@pytest.mark.parametrize("heads", [(64, 1), (64, 2), (40, 1)], ids=lambda h: f"{h[0]}q{h[1]}kv")
@pytest.mark.parametrize("D", [64, 128])
def test_large_group_decode_ignores_cache_tail(heads, D):
    """More than 16 query heads per KV head run on the tcgen05 kernel (the heads of a group are the
    rows of one query tile).  The cache past each sequence's valid length is filled with NaN: it
    must not reach the result, whichever split it falls into."""
    Hq, Hkv = heads
    B, L, dtype = 5, 3000, torch.bfloat16
    Q, K, V = qkv(2100 + Hq + D, B, Hq, Hkv, 1, L, D, dtype)
    lens = torch.tensor([1, 127, 128, 1501, 3000], dtype=torch.int32)
    Kd, Vd = K.to(DEV), V.to(DEV)
    for b in range(B):
        Kd[b, :, int(lens[b]):] = float("nan")
        Vd[b, :, int(lens[b]):] = float("nan")
    got = dense(Q.to(DEV), Kd, Vd, kv_lens=lens.to(DEV))
    assert torch.isfinite(got).all()
    assert_close(got, orc.attention(Q, K, V, kv_lens=lens), dtype, what=f"large-group decode {heads} D={D}")
