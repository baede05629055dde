"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header
declares, and the ctypes structures have the sizes the C compiler gives the header's structs."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

from attentionfuse_b200.runtime import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "attnfuse_b200.h"


def declared_functions():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"AF_API\s+[\w\s\*]+?\b(af_\w+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == names
    assert lib.af_abi_version() == 4
    assert lib.af_launch_count() >= 0


def test_struct_layouts_match_the_header(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "attnfuse_b200.h"\n'
        "int main(void) {\n"
        '  printf("%zu %zu %zu %zu\\n", sizeof(AfProblem), sizeof(AfFwdParams), sizeof(AfBwdParams), sizeof(AfDecodeParams));\n'
        '  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", offsetof(AfProblem, q), offsetof(AfProblem, status), offsetof(AfFwdParams, workspace),\n'
        "         offsetof(AfBwdParams, dv), offsetof(AfDecodeParams, partial), offsetof(AfProblem, q_bits),\n"
        "         offsetof(AfBwdParams, dq_accum), offsetof(AfDecodeParams, balanced_ctas), offsetof(AfDecodeParams, kv_pos_stride));\n"
        "  return 0;\n}\n")
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    sizes = [int(x) for x in out]
    assert sizes[:4] == [C.sizeof(_lib.AfProblem), C.sizeof(_lib.AfFwdParams), C.sizeof(_lib.AfBwdParams),
                         C.sizeof(_lib.AfDecodeParams)]
    assert sizes[4:] == [_lib.AfProblem.q.offset, _lib.AfProblem.status.offset, _lib.AfFwdParams.workspace.offset,
                         _lib.AfBwdParams.dv.offset, _lib.AfDecodeParams.partial.offset, _lib.AfProblem.q_bits.offset,
                         _lib.AfBwdParams.dq_accum.offset, _lib.AfDecodeParams.balanced_ctas.offset, _lib.AfDecodeParams.kv_pos_stride.offset]


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.af_decode_num_splits(16, 32, 8, 32768, 148, 1) == 12    # ragged lengths: 1480 CTA slots / 128 units
    assert lib.af_decode_num_splits(16, 32, 8, 32768, 148, 0) == 16    # equal lengths: 2048 CTAs = 6.9 waves of 296 slots
    assert lib.af_decode_num_splits(16, 64, 1, 32768, 148, 0) == 9     # MQA: one item per SM of the persistent kernel
    assert lib.af_decode_num_splits(1, 8, 8, 32768, 148, 0) == 64      # capped
    assert lib.af_decode_num_splits(1, 1, 1, 300, 148, 0) == 1         # fewer than 512 keys per split
    assert lib.af_decode_num_splits(16, 32, 8, 4096, 148, 1) == 8
    # invalid arguments are refused on the host, before any CUDA call
    params = _lib.AfFwdParams()
    params.p.dtype = 7
    assert lib.af_fwd(C.byref(params), None) == -1
    assert "dtype" in _lib.last_error()
    assert lib.af_fwd(None, None) == -1
    assert lib.af_decode_static(None, None) == -1


def test_misaligned_decode_workspace_is_refused_before_any_launch():
    """The combine reads ws_acc with 16-byte vectors: a ws_acc that is not 16-byte aligned is an
    invalid-argument error on the host (checked before the first CUDA call, so it runs here)."""
    lib = _lib.load()
    p = _lib.AfDecodeParams()
    p.dtype, p.B, p.H_q, p.H_kv, p.N_kv, p.D = _lib.AF_BF16, 1, 3, 1, 1536, 128
    p.sm_scale, p.num_splits = 0.088, 3
    base = 0x10000
    p.ws_m, p.ws_l, p.ws_acc = base, base + 4 * 9, base + 8 * 9      # the unpadded layout: 8-byte aligned
    assert lib.af_decode_split(C.byref(p), None) == -1
    assert "ws_acc" in _lib.last_error()
    assert lib.af_decode_combine(C.byref(p), None) == -1
    for rows in (1, 3, 9, 15, 16, 45):
        n_pad = (rows + 3) & ~3
        assert (2 * n_pad * 4) % 16 == 0


def test_int64_entry_points_return_int64():
    """Every export the header declares as int64_t is bound with a 64-bit restype."""
    lib = _lib.load()
    text = HEADER.read_text()
    wide = sorted(set(re.findall(r"AF_API\s+int64_t\s+(af_\w+)\s*\(", text)))
    assert "af_bwd_workspace_bytes" in wide and "af_fwd_workspace_bytes" in wide
    for name in wide:
        assert getattr(lib, name).restype is C.c_int64, name


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.AttnFuseLibraryError, match="no fallback"):
        _lib.load()
