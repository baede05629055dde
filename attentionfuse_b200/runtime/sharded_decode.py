"""KV-sequence-sharded decode across GPUs: the one multi-GPU path with an exchange step.

Two layouts of the sequence over G ranks:
  "contiguous"  rank r owns keys [r*L/G, (r+1)*L/G) of every (batch, kv head);
  "cyclic"      rank r owns the key blocks r, r+G, r+2G, ... of CYCLIC_BLOCK keys (what a paged
                cache that deals new blocks round-robin produces).  With per-sequence valid
                lengths the contiguous layout leaves the last ranks nearly idle (a row of length
                L/2 has no key at all on the upper half of the ranks); the cyclic layout gives every
                rank len/G keys of every row to within one block, so the step scales.
In both layouts the valid keys of a row are a prefix of the rank's local order.  Each rank runs the local
split-K decode on its slice and produces a packed partial (normalised O, LSE) of shape
(B, H_q, D+1) fp32; one all-gather (NCCL over NVLink on GPUs) places all partials in every
rank's own memory, and the gathered-combine kernel merges them there.  A rank whose slice
holds no valid key for a row contributes LSE = -inf and is ignored by the merge.
The reference is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def shard_bounds(L: int, world: int, rank: int) -> Tuple[int, int]:
    """Global key range [lo, hi) owned by `rank`; equal slices of ceil(L / world) keys."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    per = (L + world - 1) // world
    lo = min(rank * per, L)
    return lo, min(lo + per, L)


CYCLIC_BLOCK = 256


def cyclic_local_lengths(kv_lens: torch.Tensor, rank: int, world: int, block: int = CYCLIC_BLOCK) -> torch.Tensor:
    """Valid keys of each row owned by `rank` under the block-cyclic layout."""
    lens = kv_lens.to(torch.int64)
    cycle = world * block
    full, rem = lens // cycle, lens % cycle
    return (full * block + (rem - rank * block).clamp(min=0, max=block)).to(torch.int32)


def cyclic_slice(t: torch.Tensor, rank: int, world: int, block: int = CYCLIC_BLOCK) -> torch.Tensor:
    """Rank `rank`'s local cache (B, H, L/world, D) cut out of a global (B, H, L, D) tensor;
    L must be a multiple of world * block."""
    B, H, L, D = t.shape
    if L % (world * block):
        raise ValueError(f"L={L} is not a multiple of world*block={world * block}")
    return t.view(B, H, L // (world * block), world, block, D)[:, :, :, rank].reshape(B, H, L // world, D)


def local_lengths(kv_lens: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Valid keys of each batch row that fall inside [lo, hi): clamp(len - lo, 0, hi - lo)."""
    return (kv_lens.to(torch.int64) - lo).clamp(min=0, max=hi - lo).to(torch.int32)


def _cuda_partial(Q, K_local, V_local, sm_scale, bias_kind, local_lens, kv_offset, q_positions, slopes):
    from .flash_decode import run_flash_decode
    B, H_q, _, D = Q.shape
    partial = torch.empty(B, H_q, D + 1, dtype=torch.float32, device=Q.device)
    run_flash_decode(None, Q, K_local, V_local, sm_scale, bias_kind, K_local.shape[1], None,
                     kv_lens=local_lens, alibi_slopes=slopes, kv_offset=kv_offset,
                     q_positions=q_positions, partial=partial)
    return partial


def _cuda_combine(gathered, out):
    from .flash_decode import combine_gathered
    return combine_gathered(gathered, out)


def sharded_decode(Q: torch.Tensor, K_local: torch.Tensor, V_local: torch.Tensor,
                   kv_lens: Optional[torch.Tensor], L_total: int, rank: int, world: int, *,
                   sm_scale: Optional[float] = None, bias_kind: int = 0, slopes=None,
                   group=None, out: Optional[torch.Tensor] = None,
                   gather_buffer: Optional[torch.Tensor] = None,
                   local_partial: Callable = _cuda_partial, combine: Callable = _cuda_combine,
                   all_gather: Optional[Callable] = None) -> torch.Tensor:
    """Decode one token against a KV cache sharded by sequence.

    Q (B, H_q, 1, D) is replicated; K_local / V_local (B, H_kv, L_local, D) hold this rank's
    key range; kv_lens (B,) are GLOBAL valid lengths (None: all L_total keys valid).
    `local_partial`, `combine` and `all_gather` are injection points for CPU tests of the host
    logic; by default they are the CUDA kernels and torch.distributed.all_gather_into_tensor.
    The gathered partials are not inspected here (that would synchronise every step);
    `check_gathered(gather_buffer)` is the debug aid that raises on a NaN log-sum-exp.
    """
    import torch.distributed as dist
    B, H_q, _, D = Q.shape
    lo, hi = shard_bounds(L_total, world, rank)
    if K_local.shape[2] < hi - lo:
        raise ValueError(f"rank {rank} owns keys [{lo}, {hi}) but K_local holds {K_local.shape[2]}")
    if kv_lens is None:
        kv_lens = torch.full((B,), L_total, dtype=torch.int32, device=Q.device)
    lens_local = local_lengths(kv_lens, lo, hi).to(Q.device)
    q_positions = (kv_lens.to(torch.int32) - 1).to(Q.device) if bias_kind == 1 else None
    if sm_scale is None:
        sm_scale = 1.0 / (D ** 0.5)
    partial = local_partial(Q, K_local, V_local, sm_scale, bias_kind, lens_local, lo, q_positions, slopes)
    if partial.shape != (B, H_q, D + 1):
        raise RuntimeError(f"local partial has shape {tuple(partial.shape)}, expected {(B, H_q, D + 1)}")
    if gather_buffer is None:
        gather_buffer = torch.empty(world, B, H_q, D + 1, dtype=torch.float32, device=partial.device)
    if all_gather is not None:
        all_gather(gather_buffer, partial)
    elif world > 1:
        dist.all_gather_into_tensor(gather_buffer.view(world * B, H_q, D + 1), partial.contiguous(), group=group)
    else:
        gather_buffer[0].copy_(partial)
    if out is None:
        out = torch.empty_like(Q)
    combine(gather_buffer, out)
    return out


class PeerExchange:
    """One rank's end of the peer-memory exchange of decode partials.

    Multi-process use: the buffer is torch symmetric memory, so every rank can store into every
    other rank's copy over NVLink.  `peer_buffers` (a list of `world` float32 tensors on ONE
    device) replaces that for single-GPU tests of the kernels, where the "ranks" are launched
    one after another."""

    def __init__(self, world: int, rank: int, B: int, H_q: int, D: int, device, *, group=None,
                 peer_buffers=None, wait_cycles: int = 0, units: int = 0):
        import ctypes as C
        from . import _lib
        lib = _lib.load()
        self.world, self.rank, self.B, self.H_q, self.D = world, rank, B, H_q, D
        n_floats = int(lib.af_decode_exchange_bytes(world, B, H_q, D)) // 4
        if peer_buffers is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            self.buffer = symm_mem.empty(n_floats, dtype=torch.float32, device=device)
            self.buffer.zero_()
            torch.cuda.synchronize(device)
            self._handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in self._handle.buffer_ptrs]
            dist.barrier(group=group)          # every rank's buffer is zeroed before anyone pushes
        else:
            if len(peer_buffers) != world or any(t.numel() < n_floats for t in peer_buffers):
                raise ValueError("peer_buffers must hold `world` tensors of af_decode_exchange_bytes() bytes")
            self.buffer = peer_buffers[rank]
            ptrs = [t.data_ptr() for t in peer_buffers]
        self.n_floats = n_floats
        self.peer_bases = torch.tensor(ptrs, dtype=torch.int64, device=device)
        # step counter, unit counter, then one ticket word per (batch, kv head, head chunk) unit
        # for the single-launch step
        self.state = torch.zeros(2 + max(int(units), B * H_q), dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.c = _lib.AfPeerExchange(world, rank, self.peer_bases.data_ptr(), self.state.data_ptr(),
                                     self.status.data_ptr(), int(wait_cycles))

    def wait_merge(self, out: torch.Tensor) -> torch.Tensor:
        from . import _lib
        lib = _lib.load()
        with torch.cuda.device(out.device):
            rc = lib.af_decode_wait_merge(self.c, self.B, self.H_q, self.D, _lib.dtype_code(out.dtype),
                                          out.data_ptr(), _lib.strides(out), _lib.current_stream(out.device))
        _lib.check(rc, "af_decode_wait_merge")
        return out

    def sharded_step(self, params, mode: int, device) -> None:
        """One launch of the fused step (mode 3), or its push / merge half (1 / 2)."""
        import ctypes as C
        from . import _lib
        lib = _lib.load()
        with _lib.on_device(device):
            rc = lib.af_decode_sharded_step(C.byref(params), C.byref(self.c), int(mode), _lib.current_stream(device))
        _lib.check(rc, "af_decode_sharded_step")

    def check_status(self) -> None:
        """Raise if a bounded wait ran out (synchronises)."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("KV-sharded decode: a peer's partial did not arrive within the wait limit")


class ShardedDecodePlan:
    """Everything of a KV-sharded decode step that does not change from token to token, prepared
    once: local valid lengths, ALiBi query positions, split count, workspaces, the packed partial
    and the gather buffer.  `step()` then issues exactly three kernel launches and one all-gather,
    which also makes the step capturable in a CUDA graph (launch latency matters: at 8 GPUs the
    local streaming part of a 32k-token step is ~30 us)."""

    def __init__(self, B: int, H_q: int, H_kv: int, D: int, L_total: int, rank: int, world: int,
                 kv_lens: Optional[torch.Tensor], device, dtype, *, sm_scale: Optional[float] = None,
                 bias_kind: int = 0, slopes=None, group=None, layout: str = "contiguous",
                 exchange: str = "nccl", peer_exchange: Optional["PeerExchange"] = None, balanced: bool = True):
        from .flash_decode import _pick_num_splits, decode_workspace
        if exchange not in ("nccl", "p2p", "fused"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.fused = exchange == "fused"
        self.exchange = None
        self.rank, self.world, self.group = rank, world, group
        self.H_kv, self.bias_kind = H_kv, bias_kind
        self.sm_scale = sm_scale if sm_scale is not None else 1.0 / (D ** 0.5)
        if kv_lens is None:
            kv_lens = torch.full((B,), L_total, dtype=torch.int32)
        if layout == "cyclic":
            if L_total % (world * CYCLIC_BLOCK):
                raise ValueError(f"cyclic layout needs L a multiple of {world * CYCLIC_BLOCK}")
            self.lo, self.hi = 0, L_total // world
            self.lens_local = cyclic_local_lengths(kv_lens.cpu(), rank, world).to(device)
        elif layout == "contiguous":
            self.lo, self.hi = shard_bounds(L_total, world, rank)
            self.lens_local = local_lengths(kv_lens.cpu(), self.lo, self.hi).to(device)
        else:
            raise ValueError(f"unknown layout {layout!r}")
        self.q_positions = (kv_lens.to(torch.int32) - 1).to(device) if bias_kind == 1 else None
        self.slopes = None if slopes is None else slopes.to(device=device, dtype=dtype).contiguous()
        index = device.index if getattr(device, "index", None) is not None else torch.cuda.current_device()
        # position of local key j: lo + j (contiguous) or rank * block + (j / block) * world * block +
        # j % block (cyclic), so that ALiBi distances are measured on the true key axis
        self.kv_offset = self.lo if layout == "contiguous" else rank * CYCLIC_BLOCK
        self.kv_pos = dict(kv_pos_block=CYCLIC_BLOCK, kv_pos_stride=world * CYCLIC_BLOCK) if layout == "cyclic" else {}
        self.num_splits = _pick_num_splits(B, H_q, H_kv, max(self.hi - self.lo, 1), index, kv_lens is not None)
        self.balanced_ctas = 0
        rows = None
        if self.fused:
            # one launch for the whole step: every CTA must be resident at once (two per SM).  With
            # the balanced schedule those CTAs share the tiles of all sequences equally; otherwise a
            # rank's share of a 32k cache gets as many splits per unit as one wave holds.
            from .flash_decode import _sm_count, balanced_rows
            units = B * H_kv * ((H_q // H_kv + 63) // 64)
            slots = 2 * _sm_count(index)
            if balanced:
                self.balanced_ctas, self.num_splits = slots, 1
                rows = balanced_rows(B, H_q, H_kv, slots)
            else:
                self.num_splits = max(1, min(slots // units, max(1, (self.hi - self.lo) // 256)))
        self.workspace = decode_workspace(self.num_splits, B, H_q, D, device, rows=rows)
        self.partial = torch.empty(B, H_q, D + 1, dtype=torch.float32, device=device)
        self.gathered = torch.empty(world, B, H_q, D + 1, dtype=torch.float32, device=device)
        if exchange in ("p2p", "fused"):
            if peer_exchange is not None:       # buffers set up by the caller (single-GPU emulation of the ranks)
                self.exchange = peer_exchange
            elif world > 1:
                self.exchange = PeerExchange(world, rank, B, H_q, D, device, group=group)

    def check(self) -> None:
        """Raise if a bounded wait of the peer exchange ran out since the last check (synchronises;
        call it at the caller's own sync points).  After a timed-out step `out` is undefined: the
        merge does not run when a peer's rows have not arrived."""
        if self.exchange is not None:
            self.exchange.check_status()

    def step(self, Q: torch.Tensor, K_local: torch.Tensor, V_local: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """One decode step; returns `out`.  With a peer exchange (`p2p`, `fused`) a peer that does not
        deliver within the wait bound leaves `out` unwritten and sets a status word: see `check()`."""
        import torch.distributed as dist
        from .flash_decode import run_flash_decode, combine_gathered
        if self.exchange is not None and self.fused:
            # one launch: split-K, per-unit merge + push to all peers, wait for the peers, final merge
            run_flash_decode(None, Q, K_local, V_local, self.sm_scale, self.bias_kind, self.H_kv, out,
                             kv_lens=self.lens_local, alibi_slopes=self.slopes, kv_offset=self.kv_offset,
                             q_positions=self.q_positions, num_splits=self.num_splits,
                             workspace=self.workspace, exchange=self.exchange, exchange_mode=3,
                             balanced_ctas=self.balanced_ctas, **self.kv_pos)
            return out
        if self.exchange is not None:
            # two launches of the local decode (split, combine + push to all peers) and the
            # wait + merge kernel; no library collective
            run_flash_decode(None, Q, K_local, V_local, self.sm_scale, self.bias_kind, self.H_kv, None,
                             kv_lens=self.lens_local, alibi_slopes=self.slopes, kv_offset=self.kv_offset,
                             q_positions=self.q_positions, num_splits=self.num_splits,
                             workspace=self.workspace, exchange=self.exchange, **self.kv_pos)
            return self.exchange.wait_merge(out)
        run_flash_decode(None, Q, K_local, V_local, self.sm_scale, self.bias_kind, self.H_kv, None,
                         kv_lens=self.lens_local, alibi_slopes=self.slopes, kv_offset=self.kv_offset,
                         q_positions=self.q_positions, partial=self.partial, num_splits=self.num_splits,
                         workspace=self.workspace, **self.kv_pos)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered.view(-1, *self.partial.shape[1:]), self.partial,
                                        group=self.group)
        else:
            self.gathered[0].copy_(self.partial)
        return combine_gathered(self.gathered, out)


def check_gathered(gathered: torch.Tensor) -> None:
    """Host-side sanity check of gathered partials (debug aid; synchronises)."""
    lse = gathered[..., -1]
    if torch.isnan(lse).any():
        bad = torch.isnan(lse).flatten(1).any(1).nonzero().flatten().tolist()
        raise RuntimeError(f"NaN log-sum-exp in the partials of rank(s) {bad}")
