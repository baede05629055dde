"""BlockMask: compressed block-sparse mask, its builder, and the block-sparse launches.

Same data structure and builder contract as the reference
(attnfuse/runtime/block_mask.py:75-202): int32 lists, query-major ``full_kv_num`` /
``full_kv_idx`` for fully active tiles, ``kv_num_blocks`` / ``kv_indices`` for partially active
ones, and key-major ``q_num_blocks`` / ``q_indices`` (all active tiles) for the dK/dV pass.  By
default a tile with any active element counts as fully active, as in the reference, whose builder
rounds partial tiles up (so its partial lists are always empty).

Extensions:
  * every list may carry a leading head axis (``(H, n_q_blocks, ...)``) so that each head has its
    own mask; 1-D / 2-D lists as built by ``create_block_mask`` are shared by all heads.
    ``create_block_mask_per_head`` / ``BlockMask.from_dense`` build such masks from a boolean
    block grid without the reference's Python loop over tiles;
  * ``create_block_mask(..., exact=True)`` keeps partially active tiles element-exact: each one
    carries a bit matrix of its active elements, which the kernels apply to the score tile;
  * the kernels' own view of a mask: lists at 128 x 128 granularity (the tile of the tensor-core
    kernels) with bit matrices for tiles that are only partly covered, built once per mask.  A
    mask at the reference's default block size of 64 thus runs on the tensor-core kernels: four
    64-blocks share one 128-tile, and the tile's bit matrix says which quadrants are on.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from . import _lib
from .dispatch import _alibi_slopes, launch_forward

KERNEL_TILE = 128


def _compress(g: torch.Tensor):
    """Boolean (..., rows, cols) -> (counts (..., rows) int32, ascending column lists (..., rows, width) int32)."""
    counts = g.sum(-1).to(torch.int32)
    width = max(1, int(counts.max()) if counts.numel() else 1)
    # stable sort moves active columns to the front in ascending order
    order = torch.sort((~g).to(torch.uint8), dim=-1, stable=True).indices[..., :width]
    keep = torch.arange(width) < counts.unsqueeze(-1)
    return counts, (order * keep).to(torch.int32)


def _pack_bits(tiles: torch.Tensor) -> torch.Tensor:
    """Boolean (n, rows, cols) -> int64 (n, rows, ceil(cols / 64)); bit c & 63 of word c >> 6 = column c."""
    n, rows, cols = tiles.shape
    words = (cols + 63) // 64
    padded = torch.zeros(n, rows, words * 64, dtype=torch.bool)
    padded[:, :, :cols] = tiles
    weights = torch.ones(64, dtype=torch.int64) << torch.arange(64, dtype=torch.int64)   # bit 63 wraps to the sign bit
    return (padded.view(n, rows, words, 64).to(torch.int64) * weights).sum(-1)


@dataclass
class _KernelLists:
    """What a launch points the parameter block at: merged lists of all active tiles in both
    orientations, and -- when some tiles are only partly active -- the number of each tile's bit
    matrix (-1: fully active) with the matrices in both orientations."""
    block_m: int
    block_n: int
    kv_num: torch.Tensor
    kv_idx: torch.Tensor
    q_num: torch.Tensor
    q_idx: torch.Tensor
    kv_slot: Optional[torch.Tensor] = None
    q_slot: Optional[torch.Tensor] = None
    kv_bits: Optional[torch.Tensor] = None
    q_bits: Optional[torch.Tensor] = None

    def to(self, device) -> "_KernelLists":
        mv = lambda t: None if t is None else t.to(device)
        return _KernelLists(self.block_m, self.block_n, mv(self.kv_num), mv(self.kv_idx), mv(self.q_num), mv(self.q_idx),
                            mv(self.kv_slot), mv(self.q_slot), mv(self.kv_bits), mv(self.q_bits))


def _kernel_lists(active: torch.Tensor, partial: torch.Tensor, tiles_of, block_m: int, block_n: int) -> _KernelLists:
    """active / partial: boolean ([H,] nq, nk) grids; tiles_of(mask) -> boolean (n, block_m, block_n)
    element patterns of the tiles selected by `mask`, in row-major order of the grid."""
    kv_num, kv_idx = _compress(active)
    q_num, q_idx = _compress(active.transpose(-1, -2))
    out = _KernelLists(block_m, block_n, kv_num.contiguous(), kv_idx.contiguous(), q_num.contiguous(), q_idx.contiguous())
    n_part = int(partial.sum())
    if n_part == 0:
        return out
    number = torch.full(partial.shape, -1, dtype=torch.int32)
    number[partial] = torch.arange(n_part, dtype=torch.int32)
    valid = torch.arange(kv_idx.shape[-1]) < kv_num.unsqueeze(-1)
    out.kv_slot = torch.where(valid, torch.gather(number, -1, kv_idx.long()), torch.full_like(kv_idx, -1)).contiguous()
    valid = torch.arange(q_idx.shape[-1]) < q_num.unsqueeze(-1)
    out.q_slot = torch.where(valid, torch.gather(number.transpose(-1, -2), -1, q_idx.long()),
                             torch.full_like(q_idx, -1)).contiguous()
    patterns = tiles_of(partial)
    out.kv_bits = _pack_bits(patterns).contiguous()
    out.q_bits = _pack_bits(patterns.transpose(1, 2)).contiguous()
    return out


def _tile_stats(elem: torch.Tensor, block_m: int, block_n: int):
    """elem: boolean ([H,] Nq, Nk).  Returns (any, all-in-range) tile grids and the padded 5-D view
    ([H,] nq, block_m, nk, block_n)."""
    lead = elem.shape[:-2]
    n_q_len, n_k_len = elem.shape[-2:]
    nq, nk = (n_q_len + block_m - 1) // block_m, (n_k_len + block_n - 1) // block_n
    padded = torch.zeros(*lead, nq * block_m, nk * block_n, dtype=torch.bool)
    padded[..., :n_q_len, :n_k_len] = elem
    inside = torch.zeros(nq * block_m, nk * block_n, dtype=torch.bool)
    inside[:n_q_len, :n_k_len] = True
    view = padded.view(*lead, nq, block_m, nk, block_n)
    any_ = view.any(-1).any(-2)
    # elements past the sequence ends do not count against "all": the kernels never look at them
    all_ = (padded | ~inside).view(*lead, nq, block_m, nk, block_n).all(-1).all(-2)
    return any_, all_, view


@dataclass
class BlockMask:
    kv_num_blocks: torch.Tensor   # ([H,] n_q_blocks) int32, partially active tiles (empty unless exact)
    kv_indices: torch.Tensor      # ([H,] n_q_blocks, max_partial) int32
    full_kv_num: torch.Tensor     # ([H,] n_q_blocks) int32, fully active tiles
    full_kv_idx: torch.Tensor     # ([H,] n_q_blocks, max_full) int32
    q_num_blocks: torch.Tensor    # ([H,] n_kv_blocks) int32, all active tiles, key-major
    q_indices: torch.Tensor       # ([H,] n_kv_blocks, max_q) int32
    BLOCK_M: int
    BLOCK_N: int
    n_q_blocks: int
    n_kv_blocks: int
    n_active: int
    n_full: int
    kernel_lists: Optional[_KernelLists] = field(default=None, repr=False)   # what the launches use

    @property
    def per_head(self) -> bool:
        return self.full_kv_num.dim() == 2

    @property
    def exact(self) -> bool:
        return self.n_active != self.n_full

    def to(self, device) -> "BlockMask":
        moved = {f: getattr(self, f).to(device) for f in (
            "kv_num_blocks", "kv_indices", "full_kv_num", "full_kv_idx", "q_num_blocks", "q_indices")}
        return BlockMask(**moved, BLOCK_M=self.BLOCK_M, BLOCK_N=self.BLOCK_N,
                         n_q_blocks=self.n_q_blocks, n_kv_blocks=self.n_kv_blocks,
                         n_active=self.n_active, n_full=self.n_full,
                         kernel_lists=None if self.kernel_lists is None else self.kernel_lists.to(device))

    def slice_heads(self, lo: int, hi: int) -> "BlockMask":
        """The masks of heads [lo, hi) of a per-head mask (a shared mask is returned as it is): what
        a rank that owns those heads needs.  Bit-matrix numbers stay global; the matrices are shared."""
        if not self.per_head:
            return self
        cut = lambda t: t[lo:hi]
        kl = self.kernel_lists
        if kl is not None:
            opt = lambda t: None if t is None else t[lo:hi]
            kl = _KernelLists(kl.block_m, kl.block_n, cut(kl.kv_num), cut(kl.kv_idx), cut(kl.q_num), cut(kl.q_idx),
                              opt(kl.kv_slot), opt(kl.q_slot), kl.kv_bits, kl.q_bits)
        return BlockMask(cut(self.kv_num_blocks), cut(self.kv_indices), cut(self.full_kv_num), cut(self.full_kv_idx),
                         cut(self.q_num_blocks), cut(self.q_indices), self.BLOCK_M, self.BLOCK_N, self.n_q_blocks,
                         self.n_kv_blocks, int(cut(self.full_kv_num).sum() + cut(self.kv_num_blocks).sum()),
                         int(cut(self.full_kv_num).sum()), kl)

    def fill(self, p: "_lib.AfProblem", H_q: int, backward: bool = False) -> None:
        """Point a parameter block at the lists (query-major always, key-major for backward)."""
        if self.per_head and self.full_kv_num.shape[0] != H_q:
            raise ValueError(f"per-head BlockMask has {self.full_kv_num.shape[0]} heads; Q has {H_q}")
        kl = self.kernel_lists
        if kl is None:   # lists assembled by hand: every listed tile fully active, at the mask's own block size
            kl = _KernelLists(self.BLOCK_M, self.BLOCK_N, self.full_kv_num, self.full_kv_idx,
                              self.q_num_blocks, self.q_indices)
        p.mask_kind = _lib.AF_MASK_BLOCKS
        p.block_m, p.block_n = kl.block_m, kl.block_n
        p.kv_num, p.kv_idx = kl.kv_num.data_ptr(), kl.kv_idx.data_ptr()
        p.kv_num_stride_h = kl.kv_num.stride(0) if self.per_head else 0
        p.kv_idx_stride_h = kl.kv_idx.stride(0) if self.per_head else 0
        p.kv_idx_stride_q = kl.kv_idx.stride(-2)
        if kl.kv_slot is not None:
            p.kv_slot, p.kv_bits = kl.kv_slot.data_ptr(), kl.kv_bits.data_ptr()
        if backward:
            p.q_num, p.q_idx = kl.q_num.data_ptr(), kl.q_idx.data_ptr()
            p.q_num_stride_h = kl.q_num.stride(0) if self.per_head else 0
            p.q_idx_stride_h = kl.q_idx.stride(0) if self.per_head else 0
            p.q_idx_stride_k = kl.q_idx.stride(-2)
            if kl.q_slot is not None:
                p.q_slot, p.q_bits = kl.q_slot.data_ptr(), kl.q_bits.data_ptr()

    def dense_grid(self) -> torch.Tensor:
        """Boolean ([H,] n_q_blocks, n_kv_blocks) grid of active tiles (on the CPU)."""
        grid = None
        for num, idx in ((self.full_kv_num, self.full_kv_idx), (self.kv_num_blocks, self.kv_indices)):
            num, idx = num.cpu().long(), idx.cpu().long()
            g = torch.zeros(*num.shape[:-1], self.n_q_blocks, self.n_kv_blocks + 1, dtype=torch.bool)
            valid = torch.arange(idx.shape[-1]) < num.unsqueeze(-1)
            # padding slots are sent to a dump column that is cut off afterwards
            target = torch.where(valid, idx, torch.full_like(idx, self.n_kv_blocks))
            g.scatter_(-1, target, torch.ones_like(target, dtype=torch.bool))
            grid = g if grid is None else grid | g
        return grid[..., : self.n_kv_blocks]

    @staticmethod
    def _assemble(full: torch.Tensor, partial: torch.Tensor, BLOCK_M: int, BLOCK_N: int, kernel_lists, device) -> "BlockMask":
        active = full | partial
        full_num, full_idx = _compress(full)
        part_num, part_idx = _compress(partial)
        q_num, q_idx = _compress(active.transpose(-1, -2))
        return BlockMask(
            kv_num_blocks=part_num.contiguous().to(device), kv_indices=part_idx.contiguous().to(device),
            full_kv_num=full_num.contiguous().to(device), full_kv_idx=full_idx.contiguous().to(device),
            q_num_blocks=q_num.contiguous().to(device), q_indices=q_idx.contiguous().to(device),
            BLOCK_M=BLOCK_M, BLOCK_N=BLOCK_N, n_q_blocks=full.shape[-2], n_kv_blocks=full.shape[-1],
            n_active=int(active.sum()), n_full=int(full.sum()),
            kernel_lists=None if kernel_lists is None else kernel_lists.to(device))

    @staticmethod
    def from_dense(grid: torch.Tensor, BLOCK_M: int, BLOCK_N: int, device="cuda") -> "BlockMask":
        """Build from a boolean grid ([H,] n_q_blocks, n_kv_blocks) of fully active tiles."""
        grid = grid.to(torch.bool).cpu()
        none = torch.zeros_like(grid)
        if BLOCK_M % KERNEL_TILE == 0 and BLOCK_N % KERNEL_TILE == 0:
            kl = _kernel_lists(grid, none, None, BLOCK_M, BLOCK_N)
        elif KERNEL_TILE % BLOCK_M == 0 and KERNEL_TILE % BLOCK_N == 0:
            # the kernels' 128 x 128 tiles: r x c blocks of the mask share one tile; a tile with all
            # of them on is fully active, one with some of them on carries the quadrant pattern
            r, c = KERNEL_TILE // BLOCK_M, KERNEL_TILE // BLOCK_N
            lead, (nq, nk) = grid.shape[:-2], grid.shape[-2:]
            tq, tk = (nq + r - 1) // r, (nk + c - 1) // c
            padded = torch.zeros(*lead, tq * r, tk * c, dtype=torch.bool)
            padded[..., :nq, :nk] = grid
            inside = torch.zeros(tq * r, tk * c, dtype=torch.bool)
            inside[:nq, :nk] = True
            sub = padded.view(*lead, tq, r, tk, c)
            any_ = sub.any(-1).any(-2)
            all_ = (padded | ~inside).view(*lead, tq, r, tk, c).all(-1).all(-2)
            partial = any_ & ~all_
            patterns = sub.movedim(-3, -2)      # ([H,] tq, tk, r, c)

            def tiles_of(mask):
                return patterns[mask].repeat_interleave(BLOCK_M, 1).repeat_interleave(BLOCK_N, 2)
            kl = _kernel_lists(any_, partial, tiles_of, KERNEL_TILE, KERNEL_TILE)
        else:
            kl = _kernel_lists(grid, none, None, BLOCK_M, BLOCK_N)   # exact kernels, the mask's own block size
        return BlockMask._assemble(grid, none, BLOCK_M, BLOCK_N, kl, device)

    @staticmethod
    def from_elements(elem: torch.Tensor, BLOCK_M: int, BLOCK_N: int, device="cuda", exact: bool = True) -> "BlockMask":
        """Build from a boolean element mask ([H,] N_q, N_kv).  exact: partially active tiles keep
        their elements; otherwise any active element activates its whole BLOCK_M x BLOCK_N tile."""
        elem = elem.to(torch.bool).cpu()
        any_, all_, _ = _tile_stats(elem, BLOCK_M, BLOCK_N)
        if not exact:
            return BlockMask.from_dense(any_, BLOCK_M, BLOCK_N, device=device)
        full, partial = any_ & all_, any_ & ~all_
        # the kernels see the same elements at their own tile size
        k_any, k_all, k_view = _tile_stats(elem, KERNEL_TILE, KERNEL_TILE)
        k_partial = k_any & ~k_all
        tiles = k_view.movedim(-3, -2)          # ([H,] tq, tk, 128, 128)
        kl = _kernel_lists(k_any, k_partial, lambda mask: tiles[mask], KERNEL_TILE, KERNEL_TILE)
        return BlockMask._assemble(full, partial, BLOCK_M, BLOCK_N, kl, device)


def create_block_mask(mask_fn: Callable, Q_LEN: int, KV_LEN: int, BLOCK_M: int = 64,
                      BLOCK_N: int = 64, device: str = "cuda", exact: bool = False) -> BlockMask:
    """Build a BlockMask from a per-element predicate ``(q_idx, kv_idx) -> bool`` evaluated on
    broadcast index tensors.  By default a tile with at least one active element is fully active
    (the reference rounds partial tiles up: attnfuse/runtime/block_mask.py:143-154); with
    ``exact=True`` partially active tiles keep exactly the predicate's elements."""
    qi = torch.arange(Q_LEN)[:, None].expand(Q_LEN, KV_LEN)
    ki = torch.arange(KV_LEN)[None, :].expand(Q_LEN, KV_LEN)
    elem = torch.as_tensor(mask_fn(qi, ki)).to(torch.bool).expand(Q_LEN, KV_LEN)
    return BlockMask.from_elements(elem, BLOCK_M, BLOCK_N, device=device, exact=exact)


def create_block_mask_per_head(grids: torch.Tensor, BLOCK_M: int, BLOCK_N: int,
                               device: str = "cuda") -> BlockMask:
    """Per-head masks from a boolean (H, n_q_blocks, n_kv_blocks) grid of active tiles."""
    if grids.dim() != 3:
        raise ValueError("grids must have shape (H, n_q_blocks, n_kv_blocks)")
    return BlockMask.from_dense(grids, BLOCK_M, BLOCK_N, device=device)


def _check_mask(Q, K, block_mask: BlockMask):
    if not isinstance(block_mask, BlockMask):
        raise TypeError("block_mask must be an attnfuse.BlockMask")
    need_q = (Q.shape[2] + block_mask.BLOCK_M - 1) // block_mask.BLOCK_M
    need_k = (K.shape[2] + block_mask.BLOCK_N - 1) // block_mask.BLOCK_N
    if need_q != block_mask.n_q_blocks or need_k != block_mask.n_kv_blocks:
        raise ValueError(
            f"BlockMask was built for {block_mask.n_q_blocks}x{block_mask.n_kv_blocks} blocks; "
            f"Q/K need {need_q}x{need_k}")
    if block_mask.full_kv_num.device != Q.device:
        raise ValueError("BlockMask lists live on a different device than Q")


def run_block_sparse(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, block_mask: BlockMask,
                     sm_scale: float, bias_kind: int = 0, out: Optional[torch.Tensor] = None,
                     save_lse: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-sparse forward (reference: attnfuse/runtime/block_mask.py:205-271)."""
    from .dispatch import validate_qkv
    validate_qkv(Q, K, V)
    _check_mask(Q, K, block_mask)
    if out is None:
        out = torch.empty_like(Q)
    slopes = _alibi_slopes(Q.shape[1], str(Q.device), str(Q.dtype)) if bias_kind == 1 else None
    return launch_forward(Q, K, V, out, sm_scale=sm_scale, mask_kind=_lib.AF_MASK_BLOCKS,
                          bias_kind=bias_kind, slopes=slopes, save_lse=save_lse,
                          block_lists=block_mask)


def run_block_sparse_backward(Q, K, V, O, L, dO, block_mask: BlockMask, sm_scale: float,
                              bias_kind: int = 0):
    """Block-sparse backward, returns (dQ, dK, dV)
    (reference: attnfuse/runtime/block_mask.py:274-363)."""
    from .backward import launch_backward
    _check_mask(Q, K, block_mask)
    slopes = _alibi_slopes(Q.shape[1], str(Q.device), str(Q.dtype)) if bias_kind == 1 else None
    return launch_backward(Q, K, V, O, L, dO, sm_scale=sm_scale, mask_kind=_lib.AF_MASK_BLOCKS,
                           bias_kind=bias_kind, slopes=slopes, block_lists=block_mask)
