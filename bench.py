"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  Headline workload: the Llama-3-8B attention layer shape, causal + RoPE,
bf16 forward (Q [4,32,4096,128], K/V [4,8,4096,128], RoPE base 500000); a step is one forward
pass over that batch.  `value` is whole-job TFLOP/s with inputs resident in HBM (algorithmic
matmul FLOPs 4*B*H_q*D*N(N+1)/2 per step; under torchrun every rank runs its own batch, weak
scaling, no collective).  `e2e` is the same metric through the public DSL call with pinned
host buffers: host->device copies of Q/K/V and the device->host copy of O are inside the timed
region, next to the plain pinned-copy time of the same bytes (`copy_floor_ms`).  `roofline`
compares the whole step (rotation pre-pass + attention kernel) with the measured bf16 GEMM peak,
`cpu_baseline` times the reference's eager CPU path on a bounded sample of the same workload, and
`extra` carries fwd+bwd TFLOP/s, a sustained (>= 2 s) run of the headline step, decode GB/s (32k
cache, per-sequence lengths) and, under torchrun, the KV-sharded decode and a strong-scaling leg:
one problem of each prefill configuration dealt out over the ranks by batch x kv-head.

`--impl reference` times the reference algorithm on the host cores only: the reference project's
own eager functions (attnfuse.reference.naive_attention + rope_utils.apply_rope) loaded from the
unmodified install under baseline/_ref when it is there, otherwise the CPU oracle port.  The
reference project is pure Python/Triton and has no compiled CPU path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG4 = dict(B=4, H_q=32, H_kv=8, N=4096, D=128, rope_base=500000.0)
DECODE = dict(B=16, H_q=32, H_kv=8, L=32768, D=128)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the forward kernel on this workload:
# not measured by this run but taken from the ncu capture of the same workload (batch 4: 266.7 MB
# read + 81.8 MB written; profiles/fwd_tcgen05_causal_rope_bf16_d128.md), and labelled so in the
# JSON line.
FWD_KERNEL_DRAM_TRAFFIC_BYTES = 348.5e6


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return json.loads(f.read_text()), "measured"
    return FALLBACK_PEAKS, "fallback"


def causal_pairs(n: int) -> int:
    return n * (n + 1) // 2


def fwd_flops(c) -> float:
    return 4.0 * c["B"] * c["H_q"] * c["D"] * causal_pairs(c["N"])


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML in a thread of
    this process (a reading every 2 ms, so that even a timed region of a few milliseconds is
    covered), nvidia-smi as a fall-back.  Read-only: no setting of the GPU is touched."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.samples, self.max_mhz, self.stop, self.thread = [], None, threading.Event(), None
        self.nvml = None

    def _nvml_loop(self, handle):
        nv = self.nvml
        while not self.stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(mhz), int(bits)))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML orders devices by PCI bus id, CUDA may not: resolve through the UUID
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            try:
                handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.nvml = nv
            self.thread = threading.Thread(target=self._nvml_loop, args=(handle,), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.nvml is not None:
            self.stop.set()
            self.thread.join(timeout=2)
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        if self.nvml is not None:
            for mhz, bits in self.samples:
                sm.append(mhz)
                for bit, name in self.REASON_BITS.items():
                    if bits & bit:
                        reasons.add(name)
            mx = [self.max_mhz] if self.max_mhz else []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_cfg4(device, seed=4000):
    from oracle import attention_oracle as orc
    c = CFG4
    dt = torch.bfloat16
    Q = orc.randn(seed, (c["B"], c["H_q"], c["N"], c["D"]), dt)
    K = orc.randn(seed + 1, (c["B"], c["H_kv"], c["N"], c["D"]), dt)
    V = orc.randn(seed + 2, (c["B"], c["H_kv"], c["N"], c["D"]), dt)
    dO = orc.randn(seed + 3, (c["B"], c["H_q"], c["N"], c["D"]), dt)
    cos, sin = orc.build_rope_cache(c["N"], c["D"], c["rope_base"], dt)
    return Q, K, V, dO, cos, sin


def load_reference_cpu():
    """The reference project's own eager CPU functions, from the unmodified install under
    baseline/_ref, imported under an alias so that they do not collide with this repository's
    `attnfuse` import path.  Returns (naive_attention, apply_rope) or None when no install is there."""
    ref = ROOT / "baseline" / "_ref" / "attnfuse"
    if not (ref / "__init__.py").exists():
        return None
    try:
        import importlib.util
        if "attnfuse_ref" not in sys.modules:
            spec = importlib.util.spec_from_file_location("attnfuse_ref", ref / "__init__.py",
                                                          submodule_search_locations=[str(ref)])
            mod = importlib.util.module_from_spec(spec)
            sys.modules["attnfuse_ref"] = mod
            spec.loader.exec_module(mod)
        import attnfuse_ref.reference.pytorch_naive as naive
        import attnfuse_ref.rope_utils as rope
        return naive.naive_attention, rope.apply_rope
    except Exception:
        sys.modules.pop("attnfuse_ref", None)
        return None


def cpu_sample(Q, K, V, cos, sin, threads: int, budget_s: float = 0.0):
    """Time the reference's CPU path on (batch, kv head) groups of the workload (4 query heads x
    4096 x 4096 each), fp32 on the rounded bf16 inputs: the reference's own functions composed as
    its tests compose them (rotate Q and K with apply_rope, expand K/V to the query heads,
    naive_attention(causal=True)) when the install is there, the oracle port otherwise.  One group
    is always timed; with `budget_s` > 0 as many further groups as fit in that many seconds (at
    most all 32) are run and the sample's throughput is returned.
    Returns (TFLOP/s, seconds, groups, kind)."""
    from oracle import attention_oracle as orc
    torch.set_num_threads(threads)
    g = CFG4["H_q"] // CFG4["H_kv"]
    c, s = cos.float(), sin.float()
    ref = load_reference_cpu()
    flops_group = 4.0 * g * CFG4["D"] * causal_pairs(CFG4["N"])

    if ref is not None:
        naive_attention, apply_rope = ref

        def attend(q, k, v):
            n = q.shape[2]
            qr = apply_rope(q.float(), c[:n], s[:n])
            kr = apply_rope(k.float(), c[:n], s[:n])
            return naive_attention(qr, kr.expand(-1, q.shape[1], -1, -1), v.float().expand(-1, q.shape[1], -1, -1), causal=True)
    else:
        def attend(q, k, v):
            return orc.attention(q, k, v, causal=True, cos=cos, sin=sin)
    attend(Q[:1, :1, :512], K[:1, :1, :512], V[:1, :1, :512])

    def run_group(i):
        b, kv = divmod(i, CFG4["H_kv"])
        attend(Q[b:b + 1, kv * g:(kv + 1) * g], K[b:b + 1, kv:kv + 1], V[b:b + 1, kv:kv + 1])
    t0 = time.perf_counter()
    run_group(0)
    first = time.perf_counter() - t0
    total_groups = CFG4["B"] * CFG4["H_kv"]
    n = 1 if budget_s <= 0 else max(1, min(total_groups, int(budget_s / max(first, 1e-3))))
    t0 = time.perf_counter()
    for i in range(n):
        run_group(i)
    sec = time.perf_counter() - t0
    return n * flops_group / sec / 1e12, sec, n, ("reference" if ref is not None else "port")


def run_reference(args):
    """`--impl reference`: the reference's CPU path on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    Q, K, V, dO, cos, sin = make_cfg4("cpu")
    times = []
    for i in range(args.warmup + args.steps):
        tf, sec, _, kind = cpu_sample(Q, K, V, cos, sin, threads)
        if i >= args.warmup:
            times.append(sec)
        if sum(times) > 120:
            break
    g = CFG4["H_q"] // CFG4["H_kv"]
    flops = 4.0 * g * CFG4["D"] * causal_pairs(CFG4["N"])
    ms = 1e3 * sum(times) / len(times)
    value = flops / (ms * 1e-3) / 1e12
    sample = (f"1 of {CFG4['B'] * CFG4['H_kv']} (batch, kv-head) groups per step: {g} query heads x 4096 x 4096, fp32 eager; "
              "one host process whatever --gpus says, so only the N=1 ratio against it is meaningful")
    print(json.dumps({
        "impl": "reference", "metric": "causal_rope_fwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "llama3-8b attention layer, causal+RoPE forward, Q[4,32,4096,128] K/V[4,8,4096,128]",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def time_region(fn, steps: int, dist_on: bool):
    """Device time of `steps` calls, bracketed by barrier + synchronize; max over ranks (ms)."""
    import torch.distributed as dist
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    ms = torch.tensor([start.elapsed_time(end)], device="cuda")
    if dist_on:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip fwd+bwd / decode side measurements")
    ap.add_argument("--sweep", choices=["cfg2", "cfg3", "cfg5"],
                    help="time the other configurations of the baseline (one JSON line per case) instead of the bench line")
    ap.add_argument("--profile-case", choices=["fwd", "bwd", "decode", "fwd_d64"],
                    help="run three iterations of a small case of one kernel family and exit (for ncu captures)")
    args = ap.parse_args()
    if args.profile_case:
        return profile_case(args.profile_case)
    if args.sweep:
        return sweep(args.sweep)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch.distributed as dist
    import attentionfuse_b200 as af
    from attentionfuse_b200.runtime import _lib
    from attentionfuse_b200.runtime.dispatch import run_attention
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode, decode_workspace, _pick_num_splits
    from attentionfuse_b200.runtime.sharded_decode import shard_bounds, sharded_decode

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_on = world > 1
    if dist_on:
        # each rank keeps to its own share of the host cores (copy issue and launch threads of
        # eight ranks otherwise share whatever the launcher left them on)
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = max(1, len(cores) // world)
            os.sched_setaffinity(0, cores[local_rank * per:(local_rank + 1) * per] or cores)
        except (AttributeError, OSError):
            pass
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    pk, pk_kind = peaks()

    @af.attention
    def causal_rope(Q, K, V):
        return af.softmax(af.causal(af.rope(Q, K))) @ V

    Qh, Kh, Vh, dOh, cosh, sinh = make_cfg4("cpu", seed=4000 + 10 * rank)
    Qp, Kp, Vp = Qh.pin_memory(), Kh.pin_memory(), Vh.pin_memory()
    Q, K, V, dO = Qh.to(dev), Kh.to(dev), Vh.to(dev), dOh.to(dev)
    cos, sin = cosh.to(dev), sinh.to(dev)
    out = torch.empty_like(Q)
    graph = causal_rope(Q, K, V, return_graph=True)
    flops = fwd_flops(CFG4)

    def step():
        run_attention(graph, Q, K, V, cos=cos, sin=sin, out=out)

    for _ in range(args.warmup):
        step()
    launches0 = _lib.launch_count()
    with ClockSampler(local_rank) as clk:
        ms_total = time_region(step, args.steps, dist_on)
    launches = _lib.launch_count() - launches0
    ms_step = ms_total / args.steps
    value = world * flops / (ms_step * 1e-3) / 1e12
    per_gpu = flops / (ms_step * 1e-3) / 1e12

    # ---- the attention kernel alone (the RoPE pre-pass is a separate, HBM-bound launch): the same
    #      instantiation runs a plain causal graph on operands that are already rotated
    @af.attention
    def causal_only(Q, K, V):
        return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V
    from attentionfuse_b200.rope_utils import apply_rope
    Qr, Kr = apply_rope(Q, cos, sin).to(Q.dtype), apply_rope(K, cos, sin).to(K.dtype)
    graph_c = causal_only(Qr, Kr, V, return_graph=True)

    def kernel_only():
        run_attention(graph_c, Qr, Kr, V, out=out)
    for _ in range(3):
        kernel_only()
    kernel_ms = time_region(kernel_only, args.steps, dist_on) / args.steps
    kernel_tflops = flops / (kernel_ms * 1e-3) / 1e12
    del Qr, Kr

    # ---- end to end: pinned host buffers in, O back to the host, through the public call.  The
    #      step is the call pattern of a host that owns the tensors: one chunk at a time, the next
    #      chunk's host-to-device copy and the previous chunk's device-to-host copy (separate
    #      streams, PCIe is full duplex) overlapping the chunk in flight.  Every byte of Q, K, V goes
    #      up and every byte of O comes down inside the timed region of every step.
    Qd, Kd, Vd, Od = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V), torch.empty_like(Q)
    Oh = torch.empty(Q.shape, dtype=Q.dtype).pin_memory()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    # chunks: (batch row, range of kv heads with their query heads) -- contiguous blocks of the
    # (B, H, N, D) tensors, the unit the multi-GPU partition deals out.  One chunk per batch row
    # measured best among uniform chunkings (4.8 ms; four chunks per row 5.1 ms, one chunk for
    # everything 6.6 ms).  The last row goes in quarters: what cannot overlap anything is the last
    # chunk's kernel and its copy down, and a quarter row makes that tail four times shorter.
    grp, n_kv_heads = CFG4["H_q"] // CFG4["H_kv"], CFG4["H_kv"]
    chunks = [(b, 0, n_kv_heads) for b in range(Q.shape[0] - 1)]
    last_step = max(1, n_kv_heads // 4)   # eighths measured slower (5.0 - 5.1 ms against 4.75 - 4.8; whole row 4.9)
    chunks += [(Q.shape[0] - 1, h0, min(h0 + last_step, n_kv_heads)) for h0 in range(0, n_kv_heads, last_step)]
    ev_in = [torch.cuda.Event() for _ in chunks]
    ev_out = [torch.cuda.Event() for _ in chunks]

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)                      # the device buffers of the previous step are consumed
        with torch.cuda.stream(s_in):
            for i, (b, h0, h1) in enumerate(chunks):
                Qd[b, h0 * grp:h1 * grp].copy_(Qp[b, h0 * grp:h1 * grp], non_blocking=True)
                Kd[b, h0:h1].copy_(Kp[b, h0:h1], non_blocking=True)
                Vd[b, h0:h1].copy_(Vp[b, h0:h1], non_blocking=True)
                ev_in[i].record(s_in)
        for i, (b, h0, h1) in enumerate(chunks):
            cur.wait_event(ev_in[i])
            run_attention(graph, Qd[b:b + 1, h0 * grp:h1 * grp], Kd[b:b + 1, h0:h1], Vd[b:b + 1, h0:h1],
                          cos=cos, sin=sin, out=Od[b:b + 1, h0 * grp:h1 * grp])
            ev_out[i].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_out[i])
                Oh[b, h0 * grp:h1 * grp].copy_(Od[b, h0 * grp:h1 * grp], non_blocking=True)
        cur.wait_stream(s_out)                     # the step ends when the last chunk of O is on the host

    for _ in range(2):
        e2e_step()
    step()                                         # the device-resident step on the same inputs
    torch.cuda.synchronize()
    if (Oh.to(dev).float() - out.float()).abs().max().item() > 1e-3:
        raise RuntimeError("end-to-end step does not reproduce the device-resident result")
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = time_region(e2e_step, e2e_steps, dist_on) / e2e_steps
    h2d = Qp.numel() * 2 + Kp.numel() * 2 + Vp.numel() * 2
    d2h = Oh.numel() * 2

    # The floor under that number: the same bytes as plain pinned copies, one cudaMemcpyAsync per
    # tensor, up and down on their own streams at the same time, all ranks at once, no kernel.
    def copy_only():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur); s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            Qd.copy_(Qp, non_blocking=True); Kd.copy_(Kp, non_blocking=True); Vd.copy_(Vp, non_blocking=True)
        with torch.cuda.stream(s_out):
            Oh.copy_(Od, non_blocking=True)
        cur.wait_stream(s_in); cur.wait_stream(s_out)
    for _ in range(2):
        copy_only()
    copy_floor_ms = time_region(copy_only, e2e_steps, dist_on) / e2e_steps

    result = {
        "metric": "causal_rope_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama3-8b attention layer, causal+RoPE forward, Q[4,32,4096,128] K/V[4,8,4096,128], "
                               "RoPE base 5e5; every rank runs its own batch",
                   "l2": "working set 335 MB per step exceeds the 126 MB L2", "partition": f"batch x kv-head, {world} rank(s), no collective"},
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "copy_floor_ms": copy_floor_ms, "copy_floor_frac": copy_floor_ms / e2e_ms,
                "copy_floor": "the same bytes as plain pinned cudaMemcpyAsync up and down at once, all ranks together, no kernel"},
        "gpu_launches": launches,
        "clocks": clk.summary(),
        # the whole causal+RoPE step: rotation pre-pass + attention kernel, the two launches `value` times
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / pk["bf16_tflops"], "traffic": FWD_KERNEL_DRAM_TRAFFIC_BYTES,
                     "traffic_source": "from_capture (attention kernel, ncu capture of this workload; algorithmic 335.5 MB)",
                     "peak_kind": f"{pk_kind} cuBLAS bf16 burst",
                     "kernel": "rope_prepass_kernel<bf16,128> + fwd_pair_kernel<bf16,causal> (two query heads of a KV group per CTA; one step = both launches)",
                     "step_ms": ms_step, "frac_of_nominal_2250": per_gpu / 2250.0,
                     "attention_kernel_alone": {"ms": kernel_ms, "tflops": kernel_tflops,
                                                "frac": kernel_tflops / pk["bf16_tflops"]}},
    }

    extra = {}
    if not args.no_extra:
        try:
            # ---- fwd + bwd (training step of the layer): 14*B*H_q*D*P algorithmic FLOPs
            def train_step():
                q = Q.detach().requires_grad_(True); k = K.detach().requires_grad_(True); v = V.detach().requires_grad_(True)
                o = causal_rope(q, k, v, cos=cos, sin=sin)
                o.backward(dO)
            train_step()
            torch.cuda.synchronize()
            t0 = time.perf_counter(); train_step(); torch.cuda.synchronize()
            one = time.perf_counter() - t0
            n = 1 if one > 2.0 else max(2, min(10, int(4.0 / max(one, 1e-3))))
            tb = time_region(train_step, n, dist_on) / n
            fb = 3.5 * flops / (tb * 1e-3) / 1e12
            extra["fwd_bwd"] = {"tflops_per_gpu": fb, "ms_per_step": tb, "frac_of_measured_peak": fb / pk["bf16_tflops"],
                                "frac_of_nominal_2250": fb / 2250.0}
        except Exception as e:  # keep the headline line alive
            extra["fwd_bwd"] = {"error": f"{type(e).__name__}: {e}"}
        try:
            extra["decode"] = bench_decode(dev, rank, world, dist_on, pk)
        except Exception as e:
            extra["decode"] = {"error": f"{type(e).__name__}: {e}"}
        try:
            extra["strong_scaling"] = bench_strong_scaling(dev, rank, world, dist_on, pk)
        except Exception as e:
            extra["strong_scaling"] = {"error": f"{type(e).__name__}: {e}"}
        try:
            # ---- the headline step back to back for >= 2 s, clocks sampled: what the kernel sustains
            #      once the part settles under its power cap
            n_sus = max(50, int(2200.0 / ms_step))
            for _ in range(20):
                step()
            with ClockSampler(local_rank) as clk2:
                sus_ms = time_region(step, n_sus, dist_on) / n_sus
            c2 = clk2.summary()
            sus_tf = flops / (sus_ms * 1e-3) / 1e12
            extra["sustained"] = {"tflops_per_gpu": sus_tf, "ms_per_step": sus_ms, "steps": n_sus, "seconds": sus_ms * n_sus / 1e3,
                                  "sm_mhz_median": c2["sm_mhz"], "reasons": c2["reasons"],
                                  "ms_x_mhz": None if not c2["sm_mhz"] else sus_ms * c2["sm_mhz"],
                                  "frac_of_sustained_gemm_peak": sus_tf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"])}
        except Exception as e:
            extra["sustained"] = {"error": f"{type(e).__name__}: {e}"}
    result["extra"] = extra

    if rank == 0:
        try:
            threads = os.cpu_count() or 1
            tf, sec, groups, kind = cpu_sample(Qh, Kh, Vh, cosh, sinh, threads, budget_s=15.0)
            result["cpu_baseline"] = {
                "value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                "sample": f"{groups} of 32 (batch, kv-head) groups of the workload: 4 query heads x 4096 x 4096 "
                          f"causal+RoPE each, fp32 eager ({'the reference project\'s own functions' if kind == 'reference' else 'oracle port'}), {sec:.1f} s"}
        except Exception as e:
            result["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                                      "sample": f"failed: {e}"}
        print(json.dumps(result))
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


def bench_strong_scaling(dev, rank, world, dist_on, pk):
    """One problem of each prefill configuration, fixed total size, dealt out over the ranks in
    units of (batch, kv head) by runtime/partition.shard, no collective in the data path: the
    Llama-3-8B layer forward + backward (32 units), the GPT-2 geometry causal forward at N = 4096
    (48 units) and the BigBird per-head block masks forward + backward (32 units, the per-head
    lists sliced by head).  Time = max over ranks; every rank also runs the whole problem once
    (untimed) and the concatenated slices of all ranks are compared with it."""
    import numpy as np
    import torch.distributed as dist
    import attentionfuse_b200 as af
    from attentionfuse_b200.runtime import partition
    from oracle import attention_oracle as orc

    def gen(seed, shape, dt):
        g = torch.Generator(device=dev).manual_seed(seed)          # same seed, same GPU model: same bits on every rank
        return torch.randn(*shape, generator=g, device=dev, dtype=dt)

    @af.attention
    def causal_rope(Q, K, V):
        return af.softmax(af.causal(af.rope(Q, K))) @ V

    @af.attention
    def causal(Q, K, V):
        return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V

    @af.attention
    def blocks(Q, K, V):
        return af.softmax(af.block_sparse(af.scaled_dot_product(Q, K))) @ V

    out = {}

    def run_case(name, B, Hq, Hkv, N, D, dt, fn, kw_for, backward, flops):
        Q, K, V = gen(7100, (B, Hq, N, D), dt), gen(7101, (B, Hkv, N, D), dt), gen(7102, (B, Hkv, N, D), dt)
        dO = gen(7103, (B, Hq, N, D), dt) if backward else None
        grp = Hq // Hkv
        rects = partition.shard(B, Hkv, world, rank)

        def compute(rect_list, sink):
            for (b0, b1, h0, h1) in rect_list:
                q, k, v = partition.slice_qkv(Q, K, V, (b0, b1, h0, h1))
                kw = kw_for(h0 * grp, h1 * grp)
                if backward:
                    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
                    o = fn(q, k, v, **kw)
                    o.backward(dO[b0:b1, h0 * grp:h1 * grp])
                    if sink is not None:
                        sink["o"][b0:b1, h0 * grp:h1 * grp] = o.detach().float()
                        sink["dq"][b0:b1, h0 * grp:h1 * grp] = q.grad.float()
                        sink["dk"][b0:b1, h0:h1] = k.grad.float()
                        sink["dv"][b0:b1, h0:h1] = v.grad.float()
                else:
                    o = fn(q, k, v, **kw)
                    if sink is not None:
                        sink["o"][b0:b1, h0 * grp:h1 * grp] = o.float()

        def sinks():
            s = {"o": torch.zeros(B, Hq, N, D, device=dev)}
            if backward:
                s.update(dq=torch.zeros(B, Hq, N, D, device=dev), dk=torch.zeros(B, Hkv, N, D, device=dev),
                         dv=torch.zeros(B, Hkv, N, D, device=dev))
            return s
        mine, whole = sinks(), sinks()
        compute(rects, mine)                                        # this rank's slices
        compute(partition.shard(B, Hkv, 1, 0), whole)               # the whole problem on this GPU
        err = 0.0
        for key in mine:
            if dist_on:
                dist.all_reduce(mine[key])                          # slices are disjoint: the sum concatenates them
            denom = whole[key].norm().item() or 1.0
            err = max(err, (mine[key] - whole[key]).norm().item() / denom)
        del mine, whole
        for _ in range(2):
            compute(rects, None)
        n = 5
        ms = time_region(lambda: compute(rects, None), n, dist_on) / n
        ms1 = time_region(lambda: compute(partition.shard(B, Hkv, 1, 0), None), n, False) / n
        out[name] = {"units": B * Hkv, "ranks": world, "ms_per_step": ms, "tflops_aggregate": flops / (ms * 1e-3) / 1e12,
                     "ms_whole_problem_on_one_gpu": ms1, "speedup_vs_one_gpu": ms1 / ms,
                     "rel_fro_slices_vs_whole": err, "backward": backward}

    c = CFG4
    cos, sin = (t.to(dev) for t in orc.build_rope_cache(c["N"], c["D"], c["rope_base"], torch.bfloat16))
    run_case("cfg4_llama3_layer_fwd_bwd", c["B"], c["H_q"], c["H_kv"], c["N"], c["D"], torch.bfloat16, causal_rope,
             lambda h0, h1: dict(cos=cos, sin=sin), True, 3.5 * fwd_flops(c))
    run_case("cfg2_causal_n4096_fwd", 4, 12, 12, 4096, 64, torch.bfloat16, causal, lambda h0, h1: {}, False,
             4.0 * 4 * 12 * 64 * causal_pairs(4096))
    B5, H5, N5, D5, blk = 2, 16, 8192, 64, 128
    nb = N5 // blk
    grids = np.zeros((H5, nb, nb), dtype=bool)
    for h in range(H5):
        rng = np.random.default_rng(5000 + h)
        gm = grids[h]
        gm[:, :2] = True; gm[:2, :] = True
        for i in range(nb):
            gm[i, max(0, i - 1):min(nb, i + 2)] = True
            free = np.flatnonzero(~gm[i])
            gm[i, rng.choice(free, size=min(3, len(free)), replace=False)] = True
    mask = af.create_block_mask_per_head(torch.from_numpy(grids), blk, blk, device=dev)
    run_case("cfg5_bigbird_per_head_fwd_bwd", B5, H5, H5, N5, D5, torch.float16, blocks,
             lambda h0, h1: dict(block_mask=mask.slice_heads(h0, h1)), True,
             3.5 * 4.0 * B5 * D5 * blk * blk * float(grids.sum()))
    return out


def _median_ms(fn, warmup=5, iters=20):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def sweep(which: str):
    """The baseline's other configurations on one GPU, median of per-call CUDA-event times, one JSON
    line per case.  cfg2: forward sweep [4,12,N,64], six compositions, bf16 and f16.  cfg3: decode,
    three head geometries x four cache lengths, lengths U[L/2, L].  cfg5: BigBird-style per-head
    block masks [2,16,8192,64] f16, forward and forward+backward, with the all-active control."""
    import numpy as np
    import attentionfuse_b200 as af
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode, decode_workspace, _pick_num_splits
    from oracle import attention_oracle as orc
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(2000)
    pk, _ = peaks()

    def rnd(*shape, dt):
        return torch.randn(*shape, generator=gen, device=dev, dtype=dt)

    if which == "cfg2":
        B, H, D, W = 4, 12, 64, 256
        sdp = af.scaled_dot_product
        fns = {
            "dense": (af.attention(lambda Q, K, V: af.softmax(sdp(Q, K)) @ V), "dense", False),
            "causal": (af.attention(lambda Q, K, V: af.softmax(af.causal(sdp(Q, K))) @ V), "causal", False),
            "window256": (af.attention(lambda Q, K, V: af.softmax(af.sliding_window(sdp(Q, K), W)) @ V), "window", False),
            "causal+alibi": (af.attention(lambda Q, K, V: af.softmax(af.causal(af.alibi(sdp(Q, K), H))) @ V), "causal", False),
            "causal+rope": (af.attention(lambda Q, K, V: af.softmax(af.causal(af.rope(Q, K))) @ V), "causal", True),
            "causal+rope+alibi": (af.attention(lambda Q, K, V: af.softmax(af.causal(af.alibi(af.rope(Q, K), H))) @ V), "causal", True),
        }
        for dt in (torch.bfloat16, torch.float16):
            for N in (512, 1024, 2048, 4096):
                Q, K, V = rnd(B, H, N, D, dt=dt), rnd(B, H, N, D, dt=dt), rnd(B, H, N, D, dt=dt)
                cos, sin = (t.to(dev) for t in orc.build_rope_cache(N, D, 10000.0, dt))
                for name, (fn, kind, rope) in fns.items():
                    kw = dict(cos=cos, sin=sin) if rope else {}
                    ms = _median_ms(lambda: fn(Q, K, V, **kw))
                    pairs = {"dense": N * N, "causal": causal_pairs(N), "window": N * (2 * W - 1) - W * (W - 1)}[kind]
                    tf = 4.0 * B * H * D * pairs / (ms * 1e-3) / 1e12
                    print(json.dumps({"sweep": "cfg2", "dtype": str(dt).split(".")[-1], "N": N, "variant": name,
                                      "ms": round(ms, 4), "tflops": round(tf, 1),
                                      "frac_of_measured_peak": round(tf / pk["bf16_tflops"], 3)}), flush=True)
    elif which == "cfg3":
        B, D, dt = 16, 128, torch.bfloat16
        for Hq, Hkv in ((32, 8), (64, 8), (64, 1)):
            for L in (1024, 4096, 16384, 32768):
                lens = torch.randint(L // 2, L + 1, (B,), generator=gen, device=dev, dtype=torch.int32)
                n_buf = 4 if L < 32768 else 3     # rotate caches: no byte of a step is still in L2
                caches = [(rnd(B, Hkv, L, D, dt=dt), rnd(B, Hkv, L, D, dt=dt)) for _ in range(n_buf)]
                Q = rnd(B, Hq, 1, D, dt=dt)
                out = torch.empty_like(Q)
                it = [0]

                from attentionfuse_b200.runtime.flash_decode import default_balanced_ctas, balanced_rows
                S = _pick_num_splits(B, Hq, Hkv, L, 0, True)
                ctas = default_balanced_ctas(B, Hq, Hkv, L, 0)
                ws = decode_workspace(S, B, Hq, D, dev, rows=balanced_rows(B, Hq, Hkv, ctas) if ctas else None)   # allocated once, as a serving loop would
                sched = dict(balanced_ctas=ctas) if ctas else dict(num_splits=S)

                def step():
                    Kc, Vc = caches[it[0] % n_buf]; it[0] += 1
                    run_flash_decode(None, Q, Kc, Vc, 1.0 / D ** 0.5, 0, Hkv, out, kv_lens=lens, workspace=ws, **sched)
                ms = _median_ms(step)
                nbytes = 2.0 * Hkv * D * 2 * float(lens.sum().item()) + 2.0 * B * Hq * D * 2
                gbs = nbytes / (ms * 1e-3) / 1e9
                print(json.dumps({"sweep": "cfg3", "H_q": Hq, "H_kv": Hkv, "L": L, "ms": round(ms, 4),
                                  "schedule": f"balanced {ctas}" if ctas else f"{S} splits", "gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / pk["hbm_gbs"], 3)}), flush=True)
                if L == 32768 and Hkv == 8:
                    # one query row at the end of each sequence with a mask / rotation: the same
                    # split-K kernels, the mask as a range of keys, RoPE on the tiles in shared memory
                    cos, sin = (t.to(dev) for t in orc.build_rope_cache(L, D, 500000.0, dt))
                    pos = lens - 1
                    ws_split = decode_workspace(S, B, Hq, D, dev)
                    for name, mask_kind, window, rope in (("causal", 1, 0, False), ("window4096", 2, 4096, False),
                                                          ("causal+rope", 1, 0, True), ("causal+rope, rotated cache", 1, 0, 2)):
                        # keys rotated on load take the split grid, as the public call does by default
                        row_ws, row_sched = (ws_split, dict(num_splits=S)) if rope is True else (ws, sched)
                        def step_masked():
                            Kc, Vc = caches[it[0] % n_buf]; it[0] += 1
                            run_flash_decode(None, Q, Kc, Vc, 1.0 / D ** 0.5, 0, Hkv, out, kv_lens=lens,
                                             workspace=row_ws, q_positions=pos, **row_sched, mask_kind=mask_kind, window=window,
                                             cos=cos if rope else None, sin=sin if rope else None, kv_rotated=(rope == 2))
                        ms = _median_ms(step_masked)
                        keys = float(torch.clamp(lens, max=window).sum().item()) if mask_kind == 2 else float(lens.sum().item())
                        nb = 2.0 * Hkv * D * 2 * keys + 2.0 * B * Hq * D * 2
                        print(json.dumps({"sweep": "cfg3", "single_row": name, "H_q": Hq, "H_kv": Hkv, "L": L,
                                          "ms": round(ms, 4), "gbs": round(nb / (ms * 1e-3) / 1e9, 1),
                                          "frac_of_measured_hbm": round(nb / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}), flush=True)
                del caches
    else:
        B, H, N, D, blk, dt = 2, 16, 8192, 64, 128, torch.float16
        nb = N // blk
        grids = np.zeros((H, nb, nb), dtype=bool)
        for h in range(H):
            rng = np.random.default_rng(5000 + h)
            g = grids[h]
            g[:, :2] = True
            g[:2, :] = True
            for i in range(nb):
                g[i, max(0, i - 1):min(nb, i + 2)] = True
                free = np.flatnonzero(~g[i])
                if len(free):
                    g[i, rng.choice(free, size=min(3, len(free)), replace=False)] = True
        masks = {"bigbird per head": af.create_block_mask_per_head(torch.from_numpy(grids), blk, blk, device=dev),
                 "all active (control)": af.create_block_mask_per_head(torch.ones(H, nb, nb, dtype=torch.bool), blk, blk, device=dev)}
        fn = af.attention(lambda Q, K, V: af.softmax(af.block_sparse(af.scaled_dot_product(Q, K))) @ V)
        Q, K, V, dO = (rnd(B, H, N, D, dt=dt) for _ in range(4))
        Qg, Kg, Vg = (t.clone().requires_grad_(True) for t in (Q, K, V))
        for name, bm in masks.items():
            active = float(bm.dense_grid().float().mean().item())
            pairs = active * N * N
            ms_f = _median_ms(lambda: fn(Q, K, V, block_mask=bm))

            def fb():
                o = fn(Qg, Kg, Vg, block_mask=bm)
                o.backward(dO)
                Qg.grad = Kg.grad = Vg.grad = None
            ms_fb = _median_ms(fb, warmup=3, iters=10)
            print(json.dumps({"sweep": "cfg5", "mask": name, "active_fraction": round(active, 4),
                              "fwd_ms": round(ms_f, 4), "fwd_tflops": round(4.0 * B * H * D * pairs / (ms_f * 1e-3) / 1e12, 1),
                              "fwd_bwd_ms": round(ms_fb, 4),
                              "fwd_bwd_tflops": round(14.0 * B * H * D * pairs / (ms_fb * 1e-3) / 1e12, 1)}), flush=True)


def profile_case(which: str):
    """Small cases for profiler captures: tensors larger than L2 but only a few hundred MB on the
    device, three iterations, no timing.  fwd: the headline shape; bwd: the headline shape at batch 2; decode: B8 H32/8
    D128 L16384 with per-sequence lengths; fwd_d64: the GPT-2 / BERT geometry of the forward sweep
    (12 heads of 64), causal, at batch 8 and N = 8192 so that the tensors (302 MB) exceed the L2."""
    import attentionfuse_b200 as af
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode
    from oracle import attention_oracle as orc
    dev, dt = torch.device("cuda", 0), torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    @af.attention
    def causal_rope(Q, K, V):
        return af.softmax(af.causal(af.rope(Q, K))) @ V

    if which == "fwd_d64":
        @af.attention
        def causal(Q, K, V):
            return af.softmax(af.causal(af.scaled_dot_product(Q, K))) @ V
        B, H, N, D = 8, 12, 8192, 64
        Q = torch.randn(B, H, N, D, generator=g, device=dev, dtype=dt)
        K = torch.randn(B, H, N, D, generator=g, device=dev, dtype=dt)
        V = torch.randn(B, H, N, D, generator=g, device=dev, dtype=dt)
        with torch.no_grad():
            for _ in range(3):
                causal(Q, K, V)
    elif which in ("fwd", "bwd"):
        # forward: the bench's own batch (0.6 GB on the device with the rotation workspace); backward: batch 2
        B, Hq, Hkv, N, D = (CFG4["B"] if which == "fwd" else 2), CFG4["H_q"], CFG4["H_kv"], CFG4["N"], CFG4["D"]
        grad = which == "bwd"
        Q = torch.randn(B, Hq, N, D, generator=g, device=dev, dtype=dt, requires_grad=grad)
        K = torch.randn(B, Hkv, N, D, generator=g, device=dev, dtype=dt, requires_grad=grad)
        V = torch.randn(B, Hkv, N, D, generator=g, device=dev, dtype=dt, requires_grad=grad)
        dO = torch.randn(B, Hq, N, D, generator=g, device=dev, dtype=dt)
        cos, sin = (t.to(dev) for t in orc.build_rope_cache(N, D, CFG4["rope_base"], dt))
        for _ in range(3):
            o = causal_rope(Q, K, V, cos=cos, sin=sin)
            if grad:
                o.backward(dO)
                Q.grad = K.grad = V.grad = None
    else:
        B, Hq, Hkv, L, D = 8, 32, 8, 16384, 128
        Q = torch.randn(B, Hq, 1, D, generator=g, device=dev, dtype=dt)
        K = torch.randn(B, Hkv, L, D, generator=g, device=dev, dtype=dt)
        V = torch.randn(B, Hkv, L, D, generator=g, device=dev, dtype=dt)
        lens = torch.randint(L // 2, L + 1, (B,), generator=g, device=dev, dtype=torch.int32)
        out = torch.empty_like(Q)
        for _ in range(3):
            run_flash_decode(None, Q, K, V, 1.0 / D ** 0.5, 0, Hkv, out, kv_lens=lens)
    torch.cuda.synchronize()
    print("ok")


def bench_decode(dev, rank, world, dist_on, pk):
    """GQA decode at a 32k cache with per-sequence lengths in [L/2, L]: achieved HBM GB/s.
    With more than one rank also the KV-sharded step (local split-K, all-gather, merge)."""
    import torch.distributed as dist
    from oracle import attention_oracle as orc
    from attentionfuse_b200.runtime.flash_decode import run_flash_decode, decode_workspace, _pick_num_splits
    from attentionfuse_b200.runtime.sharded_decode import shard_bounds, sharded_decode
    c = DECODE
    B, Hq, Hkv, L, D = c["B"], c["H_q"], c["H_kv"], c["L"], c["D"]
    dt = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(3000)
    lens = torch.randint(L // 2, L + 1, (B,), generator=g, dtype=torch.int32)
    gen = torch.Generator(device=dev).manual_seed(3001)
    n_buf = 3   # rotate caches so that no K/V byte of a step is still in L2 from the previous one
    caches = [(torch.randn(B, Hkv, L, D, generator=gen, device=dev, dtype=dt),
               torch.randn(B, Hkv, L, D, generator=gen, device=dev, dtype=dt)) for _ in range(n_buf)]
    Q = torch.randn(B, Hq, 1, D, generator=gen, device=dev, dtype=dt)
    out = torch.empty_like(Q)
    lens_d = lens.to(dev)
    from attentionfuse_b200.runtime.flash_decode import default_balanced_ctas, balanced_rows
    S = _pick_num_splits(B, Hq, Hkv, L, dev.index or 0, True)
    ctas = default_balanced_ctas(B, Hq, Hkv, L, dev.index or 0)      # the schedule the public call picks
    ws = decode_workspace(S, B, Hq, D, dev, rows=balanced_rows(B, Hq, Hkv, ctas) if ctas else None)
    sched = dict(balanced_ctas=ctas) if ctas else dict(num_splits=S)
    sm_scale = 1.0 / D ** 0.5
    bytes_step = 2.0 * Hkv * D * 2 * float(lens.sum()) + 2.0 * B * Hq * D * 2
    it = [0]

    def step():
        Kc, Vc = caches[it[0] % n_buf]; it[0] += 1
        run_flash_decode(None, Q, Kc, Vc, sm_scale, 0, Hkv, out, kv_lens=lens_d, workspace=ws, **sched)

    for _ in range(5):
        step()
    ms = time_region(step, 30, dist_on) / 30
    gbs = bytes_step / (ms * 1e-3) / 1e9
    res = {"gbs_per_gpu": gbs, "ms_per_step": ms, "bytes_per_step": bytes_step,
           "schedule": f"balanced, {ctas} CTAs" if ctas else f"{S} splits per (batch, kv head)",
           "frac_of_measured_hbm": gbs / pk["hbm_gbs"], "frac_of_nominal_8000": gbs / 8000.0,
           "config": "B16 H32/8 D128 L32768 bf16, lengths U[L/2, L], 3 rotating caches (2.1 GB each)"}
    # CUDA-graph replay of the two launches (launch overhead matters at this step time)
    try:
        gr = torch.cuda.CUDAGraph()
        Kc, Vc = caches[0]
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            run_flash_decode(None, Q, Kc, Vc, sm_scale, 0, Hkv, out, kv_lens=lens_d, workspace=ws, **sched)
            torch.cuda.synchronize()
            with torch.cuda.graph(gr, stream=s):
                for i in range(n_buf):
                    run_flash_decode(None, Q, caches[i][0], caches[i][1], sm_scale, 0, Hkv, out, kv_lens=lens_d,
                                     workspace=ws, **sched)
        torch.cuda.synchronize()
        msg = time_region(gr.replay, 10, dist_on) / (10 * n_buf)
        res["graph_gbs_per_gpu"] = bytes_step / (msg * 1e-3) / 1e9
        res["graph_ms_per_step"] = msg
    except Exception as e:
        res["graph_error"] = f"{type(e).__name__}: {e}"

    if dist_on:
        from attentionfuse_b200.runtime.sharded_decode import ShardedDecodePlan
        from attentionfuse_b200.runtime.sharded_decode import cyclic_slice
        # block-cyclic layout of the sequence over the ranks: balanced under ragged lengths
        Kl = cyclic_slice(caches[0][0], rank, world).contiguous(); Vl = cyclic_slice(caches[0][1], rank, world).contiguous()
        plan = ShardedDecodePlan(B, Hq, Hkv, D, L, rank, world, lens, dev, dt, layout="cyclic")
        ref_out = torch.empty_like(Q)
        run_flash_decode(None, Q, caches[0][0], caches[0][1], sm_scale, 0, Hkv, ref_out, kv_lens=lens_d,
                         workspace=ws, **sched)

        def sharded():
            plan.step(Q, Kl, Vl, out)
        for _ in range(5):
            sharded()
        torch.cuda.synchronize()
        err = (out.float() - ref_out.float()).abs().max().item()
        mss = time_region(sharded, 30, True) / 30
        res["kv_sharded"] = {"world": world, "ms_per_step": mss, "speedup_vs_1gpu_step": ms / mss,
                             "aggregate_gbs": bytes_step / (mss * 1e-3) / 1e9, "local_splits": plan.num_splits, "layout": "cyclic, 256-key blocks",
                             "max_abs_vs_unsharded": err}
        try:   # fused exchange over peer memory (symmetric memory, no library collective)
            plan2 = ShardedDecodePlan(B, Hq, Hkv, D, L, rank, world, lens, dev, dt, layout="cyclic", exchange="p2p")

            def sharded_p2p():
                plan2.step(Q, Kl, Vl, out)
            for _ in range(5):
                sharded_p2p()
            torch.cuda.synchronize()
            plan2.exchange.check_status()
            err2 = (out.float() - ref_out.float()).abs().max().item()
            msp = time_region(sharded_p2p, 30, True) / 30
            res["kv_sharded_p2p"] = {"world": world, "ms_per_step": msp, "speedup_vs_1gpu_step": ms / msp,
                                     "max_abs_vs_unsharded": err2, "launches_per_step": 3}
            gs = torch.cuda.Stream()
            gs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(gs):
                for _ in range(3):
                    sharded_p2p()
            torch.cuda.current_stream().wait_stream(gs)
            torch.cuda.synchronize()
            dist.barrier()
            gr3 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr3):
                for _ in range(10):
                    sharded_p2p()
            torch.cuda.synchronize()
            dist.barrier()
            msg3 = time_region(gr3.replay, 5, True) / 50
            plan2.exchange.check_status()
            res["kv_sharded_p2p"].update({"graph_ms_per_step": msg3, "graph_speedup_vs_1gpu_graph_step":
                                          res.get("graph_ms_per_step", ms) / msg3})
        except Exception as e:
            res["kv_sharded_p2p_error"] = f"{type(e).__name__}: {e}"
        try:   # the whole step as ONE launch: split-K, per-unit merge + peer push, bounded wait, final merge
            plan3 = ShardedDecodePlan(B, Hq, Hkv, D, L, rank, world, lens, dev, dt, layout="cyclic", exchange="fused")

            def sharded_fused():
                plan3.step(Q, Kl, Vl, out)
            for _ in range(5):
                sharded_fused()
            torch.cuda.synchronize()
            plan3.exchange.check_status()
            err3 = (out.float() - ref_out.float()).abs().max().item()
            msf = time_region(sharded_fused, 30, True) / 30
            res["kv_sharded_fused"] = {"world": world, "ms_per_step": msf, "speedup_vs_1gpu_step": ms / msf,
                                       "max_abs_vs_unsharded": err3, "launches_per_step": 1, "local_splits": plan3.num_splits}
            gs = torch.cuda.Stream()
            gs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(gs):
                for _ in range(3):
                    sharded_fused()
            torch.cuda.current_stream().wait_stream(gs)
            torch.cuda.synchronize()
            dist.barrier()
            gr4 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr4):
                for _ in range(10):
                    sharded_fused()
            torch.cuda.synchronize()
            dist.barrier()
            msg4 = time_region(gr4.replay, 5, True) / 50
            plan3.exchange.check_status()
            res["kv_sharded_fused"].update({"graph_ms_per_step": msg4, "graph_speedup_vs_1gpu_graph_step":
                                            res.get("graph_ms_per_step", ms) / msg4})
        except Exception as e:
            res["kv_sharded_fused_error"] = f"{type(e).__name__}: {e}"
        try:   # the same step replayed from a CUDA graph (3 kernels + 1 all-gather per step)
            gs = torch.cuda.Stream()
            gs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(gs):
                for _ in range(3):
                    sharded()
            torch.cuda.current_stream().wait_stream(gs)
            torch.cuda.synchronize()
            gr2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr2):
                for _ in range(10):
                    sharded()
            torch.cuda.synchronize()
            msg2 = time_region(gr2.replay, 5, True) / 50
            res["kv_sharded"].update({"graph_ms_per_step": msg2, "graph_speedup_vs_1gpu_graph_step":
                                      res.get("graph_ms_per_step", ms) / msg2})
        except Exception as e:
            res["kv_sharded"]["graph_error"] = f"{type(e).__name__}: {e}"
    return res


if __name__ == "__main__":
    main()
