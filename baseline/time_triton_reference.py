"""Same-box secondary baseline: the reference's own Triton kernels timed on this GPU.

The reference package (installed unmodified under baseline/_ref, git-ignored) is imported in a
child process of its own per case, so that a Triton compile error or a crash in one case is
recorded as that case's failure text and the others still run.  Timing follows the reference's
recipe (benchmarks/bench_runner.py:118-140): warm-up calls, then one CUDA-event pair per call,
median.  With ``--impl ours`` the same cases run through this repository's package instead, with
the same harness, so the two columns are comparable.

    python baseline/time_triton_reference.py --out triton_reference.jsonl
    python baseline/time_triton_reference.py --impl ours --out triton_ours.jsonl
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

# name -> (variant, dtype, B, H_q, H_kv, N_q, N_kv, D, rope_base, backward)
CASES = {
    "cfg2_dense_n4096_bf16": ("dense", "bfloat16", 4, 12, 12, 4096, 4096, 64, None, False),
    "cfg2_causal_n4096_bf16": ("causal", "bfloat16", 4, 12, 12, 4096, 4096, 64, None, False),
    "cfg2_window256_n4096_bf16": ("window256", "bfloat16", 4, 12, 12, 4096, 4096, 64, None, False),
    "cfg2_causal_alibi_n4096_bf16": ("causal_alibi", "bfloat16", 4, 12, 12, 4096, 4096, 64, None, False),
    "cfg2_causal_rope_n4096_bf16": ("causal_rope", "bfloat16", 4, 12, 12, 4096, 4096, 64, 10000.0, False),
    "cfg2_causal_n512_bf16": ("causal", "bfloat16", 4, 12, 12, 512, 512, 64, None, False),
    "cfg4_causal_rope_fwd_bf16": ("causal_rope", "bfloat16", 4, 32, 8, 4096, 4096, 128, 500000.0, False),
    "cfg4_causal_fwd_bf16": ("causal", "bfloat16", 4, 32, 8, 4096, 4096, 128, None, False),
    "cfg4_causal_fwd_bwd_bf16": ("causal", "bfloat16", 4, 32, 8, 4096, 4096, 128, None, True),
    "cfg2_causal_fwd_bwd_n4096_f16": ("causal", "float16", 4, 12, 12, 4096, 4096, 64, None, True),
    "cfg3_decode_32q8kv_l32768_bf16": ("dense", "bfloat16", 16, 32, 8, 1, 32768, 128, None, False),
    "cfg3_decode_32q8kv_l4096_bf16": ("dense", "bfloat16", 16, 32, 8, 1, 4096, 128, None, False),
}


def unmasked_pairs(variant: str, n_q: int, n_kv: int) -> float:
    if variant.startswith("causal"):
        return n_q * (n_q + 1) / 2
    if variant == "window256":
        w = 256
        return n_q * (2 * w - 1) - w * (w - 1)
    return float(n_q) * n_kv


def run_case(name: str, impl: str, warmup: int, iters: int) -> dict:
    variant, dtype_s, B, Hq, Hkv, Nq, Nkv, D, base, backward = CASES[name]
    sys.path.insert(0, str(REF if impl == "reference" else ROOT))
    import torch
    import attnfuse as af
    from attnfuse.rope_utils import build_rope_cache

    dtype = getattr(torch, dtype_s)
    dev = "cuda"
    g = torch.Generator(device="cpu").manual_seed(1234)
    Q = torch.randn(B, Hq, Nq, D, generator=g).to(dtype).to(dev)
    K = torch.randn(B, Hkv, Nkv, D, generator=g).to(dtype).to(dev)
    V = torch.randn(B, Hkv, Nkv, D, generator=g).to(dtype).to(dev)
    kw = {}
    if variant == "dense":
        @af.attention
        def fn(Q, K, V):
            return af.softmax(af.scaled_dot_product(Q, K)) @ V
    elif variant == "causal":
        @af.attention
        def fn(Q, K, V):
            return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V
    elif variant == "window256":
        @af.attention
        def fn(Q, K, V):
            return af.softmax(af.sliding_window(af.scaled_dot_product(Q, K), 256)) @ V
    elif variant == "causal_alibi":
        @af.attention
        def fn(Q, K, V):
            return af.softmax(af.causal(af.alibi(af.scaled_dot_product(Q, K), Hq))) @ V
    elif variant == "causal_rope":
        @af.attention
        def fn(Q, K, V):
            return af.softmax(af.causal(af.rope(Q, K))) @ V
        cos, sin = build_rope_cache(Nq, D, base=base, device=dev, dtype=dtype)
        kw = {"cos": cos, "sin": sin}
    else:
        raise KeyError(variant)

    if backward:
        Q.requires_grad_(True); K.requires_grad_(True); V.requires_grad_(True)
        dO = torch.randn(B, Hq, Nq, D, generator=g).to(dtype).to(dev)

        def step():
            out = fn(Q, K, V, **kw)
            out.backward(dO)
            Q.grad = K.grad = V.grad = None
    else:
        def step():
            fn(Q, K, V, **kw)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for s, e in zip(starts, stops):
        s.record()
        step()
        e.record()
    torch.cuda.synchronize()
    ms = statistics.median(s.elapsed_time(e) for s, e in zip(starts, stops))
    pairs = unmasked_pairs(variant, Nq, Nkv)
    flops = (14.0 if backward else 4.0) * B * Hq * D * pairs
    row = {"case": name, "impl": impl, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "warmup": warmup, "iters": iters}
    if Nq == 1:
        row["gbs"] = (2.0 * B * Hkv * Nkv * D * 2 + 2.0 * B * Hq * D * 2) / (ms * 1e-3) / 1e9
    import triton
    row["torch"], row["triton"] = torch.__version__, triton.__version__
    row["package"] = str(Path(af.__file__).resolve().parent)
    return row


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("reference", "ours"), default="reference")
    ap.add_argument("--case", default=None, help="run one case in this process and print its JSON row")
    ap.add_argument("--cases", default=",".join(CASES))
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--timeout", type=int, default=300)
    ap.add_argument("--out", default=None)
    ns = ap.parse_args()
    if ns.case:
        print("ROW " + json.dumps(run_case(ns.case, ns.impl, ns.warmup, ns.iters)))
        return
    if ns.impl == "reference" and not (REF / "attnfuse").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no reference install"}))
        return
    rows = []
    for name in ns.cases.split(","):
        cmd = [sys.executable, __file__, "--impl", ns.impl, "--case", name, "--warmup", str(ns.warmup),
               "--iters", str(ns.iters)]
        env = dict(os.environ)
        env.pop("PYTHONPATH", None)
        try:
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=ns.timeout, env=env, cwd="/tmp")
            line = next((ln for ln in res.stdout.splitlines() if ln.startswith("ROW ")), None)
            if res.returncode == 0 and line:
                row = json.loads(line[4:])
            else:
                tail = (res.stderr or res.stdout).strip().splitlines()[-12:]
                row = {"case": name, "impl": ns.impl, "failed": True, "returncode": res.returncode, "tail": tail}
        except subprocess.TimeoutExpired:
            row = {"case": name, "impl": ns.impl, "failed": True, "tail": [f"timed out after {ns.timeout} s"]}
        rows.append(row)
        print(json.dumps(row), flush=True)
        if ns.out:
            with open(ns.out, "a") as f:
                f.write(json.dumps(row) + "\n")


if __name__ == "__main__":
    main()
