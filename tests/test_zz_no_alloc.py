"""The allocation-free decode entry point, af_decode_static, through the C ABI.

Some callers cannot allocate device memory at the time they decode (all memory already belongs
to their own pool, or they sit on a path where the allocator must not run).  For them the
library keeps the split-K partials in a fixed array inside its own image.  This test calls
that entry point directly with ctypes -- inputs and outputs only, no workspace -- twice in a
row with different problems, and checks each result against the regular decode path, whose
workspaces come from torch.  The second call reuses the array the first one filled, so a stale
partial leaking through would show up as a mismatch.  The file sorts last on purpose: a run
that stops at the first failure has then already executed every other test.
"""
import ctypes as C

import pytest
import torch

from attentionfuse_b200.runtime import _lib
from attentionfuse_b200.runtime.flash_decode import run_flash_decode, _pick_num_splits
from oracle import attention_oracle as orc
from tests._util import assert_close, qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCRATCH_BYTES = 4 * 1024 * 1024


def decode_static(Q, K, V, out, kv_lens=None, num_splits=0):
    """Fill AfDecodeParams by hand (no workspace pointers) and call af_decode_static."""
    lib = _lib.load()
    B, H_q, _, D = Q.shape
    p = _lib.AfDecodeParams()
    p.dtype = _lib.dtype_code(Q.dtype)
    p.B, p.H_q, p.H_kv, p.N_kv, p.D = B, H_q, K.shape[1], K.shape[2], D
    p.sm_scale, p.bias_kind, p.num_splits = 1.0 / D ** 0.5, 0, num_splits
    p.q, p.q_stride = Q.data_ptr(), _lib.strides(Q)
    p.k, p.k_stride = K.data_ptr(), _lib.strides(K)
    p.v, p.v_stride = V.data_ptr(), _lib.strides(V)
    p.kv_lens = _lib.ptr(kv_lens)
    p.o, p.o_stride = out.data_ptr(), _lib.strides(out)
    return lib.af_decode_static(C.byref(p), _lib.current_stream(Q.device))


def test_static_scratch_decode_matches_regular_path_twice():
    cases = [  # B, H_q, H_kv, L, D, dtype
        (4, 32, 8, 4096, 128, torch.bfloat16),
        (2, 16, 2, 1500, 64, torch.float16),
        (3, 9, 3, 1536, 128, torch.bfloat16),      # an odd number of partial rows
        (1, 5, 5, 1536, 128, torch.float16),
    ]
    for i, (B, Hq, Hkv, L, D, dt) in enumerate(cases):
        Q, K, V = qkv(7000 + 10 * i, B, Hq, Hkv, 1, L, D, dt)
        g = torch.Generator(device="cpu").manual_seed(70 + i)
        lens = torch.randint(L // 2, L + 1, (B,), generator=g, dtype=torch.int32)
        q, k, v, lens_d = Q.to(DEV), K.to(DEV), V.to(DEV), lens.to(DEV)
        want = torch.empty_like(q)
        # the regular entry points with torch-allocated workspaces, on the same split grid the
        # allocation-free entry point uses (the public call's default is the balanced schedule)
        run_flash_decode(None, q, k, v, 1.0 / D ** 0.5, 0, Hkv, want, kv_lens=lens_d,
                         num_splits=_pick_num_splits(B, Hq, Hkv, L, 0, True))
        got = torch.full_like(q, float("nan"))
        rc = decode_static(q, k, v, got, kv_lens=lens_d)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        # same kernels, same split count, same arithmetic: identical bits
        assert torch.equal(got, want), f"case {i}: static-scratch decode differs from the regular path"
        assert_close(got, orc.attention(Q, K, V, kv_lens=lens), dt, what=f"case {i} vs oracle")


def test_static_scratch_rejects_oversized_problem():
    B, Hq, Hkv, L, D = 64, 64, 8, 512, 128
    Q, K, V = (torch.zeros(B, h, n, D, dtype=torch.bfloat16, device=DEV) for h, n in ((Hq, 1), (Hkv, L), (Hkv, L)))
    out = torch.zeros_like(Q)
    splits = 4
    assert splits * B * Hq * (D + 2) * 4 > SCRATCH_BYTES      # rows are a multiple of 4 here: no padding
    rc = decode_static(Q, K, V, out, num_splits=splits)
    assert rc == -4                                   # AF_ERR_WORKSPACE, nothing launched
    assert "exceeds the built-in scratch" in _lib.last_error()
