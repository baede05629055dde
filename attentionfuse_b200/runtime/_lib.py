"""ctypes binding of the C-ABI shared library (include/attnfuse_b200.h).

The library is the only compute path: if it is missing or fails to load, every launch
raises -- there is no eager or CPU fallback.  Structures here mirror the header field for
field; `tests/test_abi.py` checks sizes and exported symbols against the header.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Optional, Sequence

import os

# ATTNFUSE_B200_LIBRARY points at a build of the library kept somewhere else
LIB_PATH = Path(os.environ.get("ATTNFUSE_B200_LIBRARY") or
                Path(__file__).resolve().parent.parent / "csrc" / "libattnfuse_b200.so")

AF_F16, AF_BF16, AF_F32 = 0, 1, 2
AF_MASK_FULL, AF_MASK_CAUSAL, AF_MASK_WINDOW, AF_MASK_BLOCKS = 0, 1, 2, 3
AF_BIAS_NONE, AF_BIAS_ALIBI, AF_BIAS_ADDITIVE = 0, 1, 2
AF_NORM_SOFTMAX, AF_NORM_RELU = 0, 1
AF_FAMILY_AUTO, AF_FAMILY_FFMA, AF_FAMILY_TCGEN05 = 0, 1, 2
AF_STATUS_OK, AF_STATUS_WAIT_TIMEOUT = 0, 1

I32, I64, F32, PTR = C.c_int32, C.c_int64, C.c_float, C.c_void_p
S4, S3 = I64 * 4, I64 * 3


class AfProblem(C.Structure):
    _fields_ = [
        ("dtype", I32), ("family", I32),
        ("B", I32), ("H_q", I32), ("H_kv", I32), ("N_q", I32), ("N_kv", I32), ("D", I32),
        ("sm_scale", F32),
        ("mask_kind", I32), ("window", I32), ("bias_kind", I32), ("norm_kind", I32), ("rope", I32),
        ("block_m", I32), ("block_n", I32),
        ("q", PTR), ("q_stride", S4),
        ("k", PTR), ("k_stride", S4),
        ("v", PTR), ("v_stride", S4),
        ("slopes", PTR),
        ("bias", PTR), ("bias_stride", S4),
        ("cos", PTR), ("sin", PTR), ("rope_stride_n", I64),
        ("kv_num", PTR), ("kv_idx", PTR),
        ("kv_num_stride_h", I64), ("kv_idx_stride_h", I64), ("kv_idx_stride_q", I64),
        ("q_num", PTR), ("q_idx", PTR),
        ("q_num_stride_h", I64), ("q_idx_stride_h", I64), ("q_idx_stride_k", I64),
        ("status", PTR),
        ("q_offset", I32),
        ("kv_slot", PTR), ("q_slot", PTR), ("kv_bits", PTR), ("q_bits", PTR),
    ]


class AfFwdParams(C.Structure):
    _fields_ = [("p", AfProblem), ("o", PTR), ("o_stride", S4), ("lse", PTR), ("lse_stride", S3),
                ("workspace", PTR), ("workspace_bytes", I64)]


class AfBwdParams(C.Structure):
    _fields_ = [
        ("p", AfProblem),
        ("o", PTR), ("o_stride", S4),
        ("d_o", PTR), ("do_stride", S4),
        ("lse", PTR), ("lse_stride", S3),
        ("delta", PTR),
        ("dq", PTR), ("dq_stride", S4),
        ("dk", PTR), ("dk_stride", S4),
        ("dv", PTR), ("dv_stride", S4),
        ("workspace", PTR), ("workspace_bytes", I64),
        ("workspace_holds_rotated", I32),
        ("dq_accum", PTR), ("dq_accum_bytes", I64),
    ]


class AfDecodeParams(C.Structure):
    _fields_ = [
        ("dtype", I32),
        ("B", I32), ("H_q", I32), ("H_kv", I32), ("N_kv", I32), ("D", I32),
        ("sm_scale", F32), ("bias_kind", I32), ("num_splits", I32),
        ("q", PTR), ("q_stride", S4),
        ("k", PTR), ("k_stride", S4),
        ("v", PTR), ("v_stride", S4),
        ("slopes", PTR), ("kv_lens", PTR), ("q_positions", PTR), ("kv_offset", I32),
        ("ws_m", PTR), ("ws_l", PTR), ("ws_acc", PTR),
        ("o", PTR), ("o_stride", S4),
        ("partial", PTR), ("status", PTR),
        ("mask_kind", I32), ("window", I32), ("rope", I32), ("q_position_p1", I32),
        ("cos", PTR), ("sin", PTR), ("rope_stride_n", I64),
        ("balanced_ctas", I32),
        ("kv_pos_block", I32), ("kv_pos_stride", I32),
    ]


class AfPeerExchange(C.Structure):
    _fields_ = [("world", I32), ("rank", I32), ("peer_bases", PTR), ("state", PTR), ("status", PTR),
                ("wait_cycles", I64)]


EXPORTS = ("af_fwd", "af_fwd_workspace_bytes", "af_bwd", "af_bwd_workspace_bytes", "af_bwd_dq_accum_bytes", "af_decode_split", "af_decode_combine", "af_decode_static", "af_decode_exchange_bytes", "af_decode_combine_push", "af_decode_wait_merge", "af_decode_sharded_step",
           "af_decode_combine_gathered", "af_decode_num_splits", "af_query_family",
           "af_launch_count", "af_last_error", "af_abi_version")

_lock = threading.Lock()
_lib: Optional[C.CDLL] = None


class AttnFuseLibraryError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load the shared library once; raise loudly if it has not been built."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise AttnFuseLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m attentionfuse_b200.csrc.build` "
                "(there is no fallback path)")
        lib = C.CDLL(str(LIB_PATH))
        lib.af_fwd.argtypes = [C.POINTER(AfFwdParams), PTR]
        lib.af_fwd_workspace_bytes.argtypes = [C.POINTER(AfFwdParams)]
        lib.af_fwd_workspace_bytes.restype = I64
        lib.af_bwd.argtypes = [C.POINTER(AfBwdParams), PTR]
        lib.af_bwd_workspace_bytes.argtypes = [C.POINTER(AfBwdParams)]
        lib.af_bwd_workspace_bytes.restype = I64
        lib.af_bwd_dq_accum_bytes.argtypes = [C.POINTER(AfBwdParams)]
        lib.af_bwd_dq_accum_bytes.restype = I64
        lib.af_decode_split.argtypes = [C.POINTER(AfDecodeParams), PTR]
        lib.af_decode_combine.argtypes = [C.POINTER(AfDecodeParams), PTR]
        lib.af_decode_exchange_bytes.argtypes = [I32, I32, I32, I32]
        lib.af_decode_exchange_bytes.restype = I64
        lib.af_decode_combine_push.argtypes = [C.POINTER(AfDecodeParams), C.POINTER(AfPeerExchange), PTR]
        lib.af_decode_combine_push.restype = I32
        lib.af_decode_wait_merge.argtypes = [C.POINTER(AfPeerExchange), I32, I32, I32, I32, PTR, C.POINTER(I64), PTR]
        lib.af_decode_wait_merge.restype = I32
        lib.af_decode_sharded_step.argtypes = [C.POINTER(AfDecodeParams), C.POINTER(AfPeerExchange), I32, PTR]
        lib.af_decode_sharded_step.restype = I32
        lib.af_decode_static.argtypes = [C.POINTER(AfDecodeParams), PTR]
        lib.af_decode_static.restype = I32
        lib.af_decode_combine_gathered.argtypes = [PTR, I32, I32, I32, I32, I32, PTR, C.POINTER(I64), PTR]
        lib.af_decode_num_splits.argtypes = [I32, I32, I32, I32, I32, I32]
        lib.af_query_family.argtypes = [C.POINTER(AfProblem), I32]
        for name in ("af_fwd", "af_bwd", "af_decode_split", "af_decode_combine",
                     "af_decode_combine_gathered", "af_decode_num_splits", "af_query_family",
                     "af_abi_version"):
            getattr(lib, name).restype = I32
        lib.af_launch_count.restype = I64
        lib.af_last_error.restype = C.c_char_p
        _lib = lib
        return lib


def last_error() -> str:
    return load().af_last_error().decode(errors="replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = last_error()
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        if rc == -2:
            raise NotImplementedError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed ({rc}): {msg}")


def launch_count() -> int:
    return int(load().af_launch_count())


# --------------------------------------------------------------------------------------
# helpers to fill the structures from torch tensors
# --------------------------------------------------------------------------------------
def dtype_code(dtype) -> int:
    import torch
    try:
        return {torch.float16: AF_F16, torch.bfloat16: AF_BF16, torch.float32: AF_F32}[dtype]
    except KeyError:
        raise NotImplementedError(f"dtype {dtype} has no kernel instantiation") from None


def ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def strides(t, n: int = 4):
    return (I64 * n)(*[int(s) for s in t.stride()])


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def on_device(device):
    """Context that makes `device` current for a launch; free when it already is (the usual
    case), a torch.cuda.device switch otherwise."""
    import torch
    if device.index is None or torch.cuda.current_device() == device.index:
        return _NO_SWITCH
    return torch.cuda.device(device)


def current_stream(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream
