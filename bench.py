#!/usr/bin/env python
"""Benchmark of the operator path on B200.

One step = one pass of the Llama-3-8B memory-bound operators over a batch of 8192 tokens, bf16:
RMSNorm over hidden 4096 (weight, eps 1e-6), RoPE on Q[8192,32,128] and K[8192,8,128]
(theta 500000) and SwiGLU on [8192,14336] — four kernel launches through the C ABI.
`value` is algorithmic GB/s (inputs read once + outputs written once) with inputs resident in
HBM; `e2e` is the same metric through the host-tensor call path with pinned host buffers and the
host<->device copies inside the timed region.  With N ranks every rank owns its own batch
(data-parallel, no collective on the data path): weak scaling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`--impl reference` times the reference's CPU path for the same workload on the host cores
(the torch-CPU restatement in oracle/, since the SOPHGO cmodel emulator cannot be installed).
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

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT / "tilelang-tpu_b200"), str(ROOT)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

# DRAM bytes one SwiGLU launch moves per token, from one ncu capture of the 4096-token case
# (301.8 MB for 4096 tokens; 86 016 algorithmic bytes per token - the part of the output still
# dirty in L2 when the kernel ends is not counted).  Traffic
# grows in proportion to the token count, so a launch is scaled from it.
SWIGLU_DRAM_BYTES_PER_TOKEN = 301.8e6 / 4096

METRIC = "GEMM/attn TFLOP/s and norm/RoPE GB/s vs B200 roofline at 1/2/4/8 GPUs"
WORKLOAD = ("llama3-8b memory-bound ops, bf16, 8192 tokens: rmsnorm[8192x4096] + "
            "rope(Q[8192,32,128],K[8192,8,128]) + swiglu[8192x14336]")
FALLBACK_HBM_GBS = 6650.0


# ------------------------------------------------------------------------------------------
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    """HBM GB/s (and the bf16 burst figure for kernels timed alone) measured on this pool."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "note": "of measured"}
        except Exception:
            pass
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "note": "of fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        inside = [r for t, r in self.rows if self.t0 is not None and self.t0 - 0.05 <= t <= self.t1 + 0.15]
        rows = inside or [r for _, r in self.rows]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                smax.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "samples_in_timed_region": len(inside)}


# ------------------------------------------------------------------------------------------
def cpu_pass(w, O):
    """One pass of the workload through the CPU restatement; returns nothing (timing only)."""
    O.rmsnorm(w["x"], w["weight"], eps=w["eps"])
    O.rope(w["q"], w["cos"], w["sin"])
    O.rope(w["k"], w["cos"], w["sin"])
    O.swiglu(w["gate"], w["up"])


def time_cpu(w, total_bytes, reps=3):
    import oracle.ops as O      # the checker, timed here as the CPU baseline only
    cpu_pass(w, O)              # warm-up
    best = float("inf")
    for _ in range(reps):
        t = time.perf_counter()
        cpu_pass(w, O)
        best = min(best, time.perf_counter() - t)
    return total_bytes / best / 1e9, best


def run_reference(args, rank):
    """Reference arm: the reference's CPU path for this workload on the host cores."""
    if rank != 0:
        return
    from tilelang import workloads
    w = workloads.llama8b_memory_ops()
    total = sum(workloads.llama8b_algorithmic_bytes().values())
    import oracle.ops as O
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_pass(w, O)
    steps = max(1, min(args.steps, 5))
    t = time.perf_counter()
    for _ in range(steps):
        cpu_pass(w, O)
    dt = (time.perf_counter() - t) / steps
    gbs = total / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens": 8192},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} full passes of the 8192-token workload "
                                   "(torch-CPU restatement of the demos' check functions; the "
                                   "reference's cmodel emulator is not installable)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per GPU (default: the named config)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true",
                    help="skip the per-kernel section (GEMM bf16/FP8, FlashAttention, MLA decode)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from tilelang import ops, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    tokens = args.tokens
    w = workloads.llama8b_memory_ops(tokens=tokens, seed=1 + rank)   # each rank owns its own batch
    alg = workloads.llama8b_algorithmic_bytes(tokens=tokens)
    bytes_per_step = sum(alg.values())

    d = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    y = torch.empty_like(d["x"])
    qo = torch.empty_like(d["q"])
    ko = torch.empty_like(d["k"])
    so = torch.empty_like(d["gate"])

    def step(ev=None):
        ops.rmsnorm(d["x"], y, d["weight"], eps=w["eps"])
        ops.rope(d["q"], d["cos"], d["sin"], qo)
        ops.rope(d["k"], d["cos"], d["sin"], ko)
        if ev is not None:
            ev[0].record()
        ops.swiglu(d["gate"], d["up"], so)
        if ev is not None:
            ev[1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)

    # events bracket the dominant kernel (SwiGLU, 70% of the bytes) inside the timed region
    n_ev = min(steps, 512)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ev)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = ops.launch_count()
    if sampler:
        sampler.mark_begin()
    start.record()
    for i in range(steps):
        step(evs[i] if i < n_ev else None)
    end.record()
    barrier()
    if sampler:
        sampler.mark_end()
    launches = ops.launch_count() - launches0
    ms_total = start.elapsed_time(end)
    swiglu_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    clocks = sampler.stop() if sampler else None

    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: pinned host tensors in, results back on the host, every step ----------
    hin = {k: w[k].pin_memory() for k in ("x", "weight", "q", "k", "cos", "sin", "gate", "up")}
    hout = {"y": torch.empty_like(w["x"]).pin_memory(), "qo": torch.empty_like(w["q"]).pin_memory(),
            "ko": torch.empty_like(w["k"]).pin_memory(), "so": torch.empty_like(w["gate"]).pin_memory()}
    h2d = sum(v.numel() * v.element_size() for v in hin.values())
    d2h = sum(v.numel() * v.element_size() for v in hout.values())

    # Three streams and two sets of device buffers: the host->device copy of step i+1 and the
    # device->host copy of step i-1 run while step i computes (PCIe is full duplex).  Every step's copies
    # are inside the timed region; nothing is reused from one step to the next.
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    din = [{k: torch.empty_like(v, device=dev) for k, v in hin.items()} for _ in range(2)]
    dout = [{"y": torch.empty_like(y), "qo": torch.empty_like(qo), "ko": torch.empty_like(ko), "so": torch.empty_like(so)}
            for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps_run(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_cmp[b])            # the step that last read these inputs has computed
                for k, v in hin.items():
                    din[b][k].copy_(v, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[b])
                if i >= 2:
                    s_cmp.wait_event(ev_out[b])           # its previous results are on the host
                dd, oo = din[b], dout[b]
                ops.rmsnorm(dd["x"], oo["y"], dd["weight"], eps=w["eps"])
                ops.rope(dd["q"], dd["cos"], dd["sin"], oo["qo"])
                ops.rope(dd["k"], dd["cos"], dd["sin"], oo["ko"])
                ops.swiglu(dd["gate"], dd["up"], oo["so"])
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                for k in ("y", "qo", "ko", "so"):
                    hout[k].copy_(dout[b][k], non_blocking=True)
                ev_out[b].record(s_out)
        for st in (s_in, s_cmp, s_out):
            torch.cuda.current_stream().wait_stream(st)

    e2e_steps = max(2, min(steps, 20))
    e2e_steps_run(2)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for st in (s_in, s_cmp, s_out):
        st.wait_event(s2)
    e2e_steps_run(e2e_steps)
    e2.record()
    barrier()
    t2 = torch.tensor([s2.elapsed_time(e2)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item()) / e2e_steps
    e2e_value = world * bytes_per_step / (e2e_ms * 1e-3) / 1e9

    # hand the big buffers back before the per-kernel section allocates its own
    del hin, hout, din, dout, d, y, qo, ko, so
    torch.cuda.empty_cache()
    peaks = measured_peaks()
    kernels = None
    if not args.no_kernels:
        import kernel_bench
        kernels = kernel_bench.run_all(dev, rank, world, peaks)

    if rank == 0:
        peak, peak_kind = peaks["hbm_gbs"], peaks["note"].replace("of ", "")
        achieved = alg["swiglu"] / (swiglu_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": tokens, "parallelism": f"dp{world}",
                       "l2": "per-step working set 1.0 GB > 126 MB L2 (inputs larger than L2, no flush)",
                       "bytes_per_step_per_gpu": bytes_per_step},
            "roofline": {"bound": "hbm", "kernel": "swiglu_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                         "traffic": SWIGLU_DRAM_BYTES_PER_TOKEN * tokens,
                         "traffic_source": "dram__bytes of one ncu capture at 4096 tokens, scaled by the token count",
                         "avg_launch_ms": swiglu_ms},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if kernels is not None:
            line["kernels"] = kernels
        if world == 1 and not args.no_cpu_baseline:
            cpu_gbs, cpu_s = time_cpu(w, bytes_per_step)
            line["cpu_baseline"] = {
                "value": cpu_gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"best of 3 full passes of the same 8192-token workload ({cpu_s:.2f} s per pass)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
