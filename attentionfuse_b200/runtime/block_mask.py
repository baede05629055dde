"""BlockMask: compressed block-sparse mask, its builder, and the block-sparse launches.

Same data structure and builder contract as the reference
(attnfuse/runtime/block_mask.py:75-202): int32 lists, query-major ``full_kv_num`` /
``full_kv_idx`` (plus the always-empty partial lists ``kv_num_blocks`` / ``kv_indices``,
because tiles with any active element are rounded up to fully active) and key-major
``q_num_blocks`` / ``q_indices`` for the dK/dV pass.

Extension: every list may carry a leading head axis (``(H, n_q_blocks, ...)``) so that each
head has its own mask; 1-D / 2-D lists as built by ``create_block_mask`` are shared by all
heads.  ``create_block_mask_per_head`` / ``BlockMask.from_dense`` build such masks from a
boolean block grid without the reference's Python loop over tiles.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _lib
from .dispatch import _alibi_slopes, launch_forward


@dataclass
class BlockMask:
    kv_num_blocks: torch.Tensor   # ([H,] n_q_blocks) int32, partial tiles (always 0)
    kv_indices: torch.Tensor      # ([H,] n_q_blocks, max_partial) int32
    full_kv_num: torch.Tensor     # ([H,] n_q_blocks) int32
    full_kv_idx: torch.Tensor     # ([H,] n_q_blocks, max_full) int32
    q_num_blocks: torch.Tensor    # ([H,] n_kv_blocks) int32
    q_indices: torch.Tensor       # ([H,] n_kv_blocks, max_q) int32
    BLOCK_M: int
    BLOCK_N: int
    n_q_blocks: int
    n_kv_blocks: int
    n_active: int
    n_full: int

    @property
    def per_head(self) -> bool:
        return self.full_kv_num.dim() == 2

    def to(self, device) -> "BlockMask":
        moved = {f: getattr(self, f).to(device) for f in (
            "kv_num_blocks", "kv_indices", "full_kv_num", "full_kv_idx", "q_num_blocks", "q_indices")}
        return BlockMask(**moved, BLOCK_M=self.BLOCK_M, BLOCK_N=self.BLOCK_N,
                         n_q_blocks=self.n_q_blocks, n_kv_blocks=self.n_kv_blocks,
                         n_active=self.n_active, n_full=self.n_full)

    def fill(self, p: "_lib.AfProblem", H_q: int, backward: bool = False) -> None:
        """Point a parameter block at the lists (query-major always, key-major for backward)."""
        if self.per_head and self.full_kv_num.shape[0] != H_q:
            raise ValueError(f"per-head BlockMask has {self.full_kv_num.shape[0]} heads; Q has {H_q}")
        p.mask_kind = _lib.AF_MASK_BLOCKS
        p.block_m, p.block_n = self.BLOCK_M, self.BLOCK_N
        num, idx = self.full_kv_num, self.full_kv_idx
        p.kv_num, p.kv_idx = num.data_ptr(), idx.data_ptr()
        p.kv_num_stride_h = num.stride(0) if self.per_head else 0
        p.kv_idx_stride_h = idx.stride(0) if self.per_head else 0
        p.kv_idx_stride_q = idx.stride(-2)
        if backward:
            qn, qi = self.q_num_blocks, self.q_indices
            p.q_num, p.q_idx = qn.data_ptr(), qi.data_ptr()
            p.q_num_stride_h = qn.stride(0) if self.per_head else 0
            p.q_idx_stride_h = qi.stride(0) if self.per_head else 0
            p.q_idx_stride_k = qi.stride(-2)

    def dense_grid(self) -> torch.Tensor:
        """Boolean ([H,] n_q_blocks, n_kv_blocks) grid of active tiles (on the CPU)."""
        num, idx = self.full_kv_num.cpu().long(), self.full_kv_idx.cpu().long()
        grid = torch.zeros(*num.shape[:-1], self.n_q_blocks, self.n_kv_blocks + 1, dtype=torch.bool)
        valid = torch.arange(idx.shape[-1]) < num.unsqueeze(-1)
        # padding slots are sent to a dump column that is cut off afterwards
        target = torch.where(valid, idx, torch.full_like(idx, self.n_kv_blocks))
        grid.scatter_(-1, target, torch.ones_like(target, dtype=torch.bool))
        return grid[..., : self.n_kv_blocks]

    @staticmethod
    def from_dense(grid: torch.Tensor, BLOCK_M: int, BLOCK_N: int, device="cuda") -> "BlockMask":
        """Build from a boolean grid ([H,] n_q_blocks, n_kv_blocks) of active tiles."""
        grid = grid.to(torch.bool).cpu()
        n_q, n_kv = grid.shape[-2], grid.shape[-1]

        def compress(g):
            counts = g.sum(-1).to(torch.int32)
            width = max(1, int(counts.max()) if counts.numel() else 1)
            # stable sort moves active columns to the front in ascending order
            order = torch.sort((~g).to(torch.uint8), dim=-1, stable=True).indices[..., :width]
            keep = torch.arange(width) < counts.unsqueeze(-1)
            return counts, (order * keep).to(torch.int32)

        full_num, full_idx = compress(grid)
        q_num, q_idx = compress(grid.transpose(-1, -2))
        lead = grid.shape[:-2]
        zeros_num = torch.zeros(*lead, n_q, dtype=torch.int32)
        zeros_idx = torch.zeros(*lead, n_q, 1, dtype=torch.int32)
        total = int(full_num.sum())
        return BlockMask(
            kv_num_blocks=zeros_num.to(device), kv_indices=zeros_idx.to(device),
            full_kv_num=full_num.contiguous().to(device), full_kv_idx=full_idx.contiguous().to(device),
            q_num_blocks=q_num.contiguous().to(device), q_indices=q_idx.contiguous().to(device),
            BLOCK_M=BLOCK_M, BLOCK_N=BLOCK_N, n_q_blocks=n_q, n_kv_blocks=n_kv,
            n_active=total, n_full=total)


def create_block_mask(mask_fn: Callable, Q_LEN: int, KV_LEN: int, BLOCK_M: int = 64,
                      BLOCK_N: int = 64, device: str = "cuda") -> BlockMask:
    """Build a BlockMask from a per-element predicate ``(q_idx, kv_idx) -> bool`` evaluated on
    broadcast index tensors.  A tile with at least one active element is fully active (the
    reference rounds partial tiles up: attnfuse/runtime/block_mask.py:143-154)."""
    n_q = (Q_LEN + BLOCK_M - 1) // BLOCK_M
    n_kv = (KV_LEN + BLOCK_N - 1) // BLOCK_N
    qi = torch.arange(Q_LEN)[:, None].expand(Q_LEN, KV_LEN)
    ki = torch.arange(KV_LEN)[None, :].expand(Q_LEN, KV_LEN)
    elem = torch.as_tensor(mask_fn(qi, ki)).to(torch.bool).expand(Q_LEN, KV_LEN)
    padded = torch.zeros(n_q * BLOCK_M, n_kv * BLOCK_N, dtype=torch.bool)
    padded[:Q_LEN, :KV_LEN] = elem
    grid = padded.view(n_q, BLOCK_M, n_kv, BLOCK_N).any(dim=3).any(dim=1)
    return BlockMask.from_dense(grid, BLOCK_M, BLOCK_N, device=device)


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
