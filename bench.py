#!/usr/bin/env python
"""Benchmark of the operator path on B200.

One step = one pass of the Llama-3-8B memory-bound operators over ONE batch of 8192 tokens, bf16:
RMSNorm over hidden 4096 (weight, eps 1e-6), RoPE on Q[8192,32,128] and K[8192,8,128]
(theta 500000) and SwiGLU on [8192,14336] - four kernels of the library per step.
With N ranks the rows (tokens) of that one batch are split over the GPUs, 8192/N each (strong
scaling); no collective is on the data path, and the all-gather of the four outputs is timed
separately (`ms_with_output_gather`).  `value` is algorithmic GB/s of the whole batch (inputs read
once + outputs written once) with inputs resident in HBM, device time, max over ranks; `e2e` is the
same metric through `tilelang.compile(...)` programs called with pinned HOST tensors, the
host<->device copies inside the timed region.

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
TOKENS = 8192
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
def config_for(world: int, tokens: int = TOKENS) -> dict:
    """The `config` object, identical in both arms."""
    return {"workload": WORKLOAD, "tokens": tokens, "sharding": f"rows (tokens) split over {world} GPU(s), {tokens // world} each",
            "l2": "every rank rotates over input sets that together exceed 1.0 GB (> 126 MB L2); no flush"}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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
    """Reference arm: the reference's CPU path for this workload on the host cores (rank 0 only)."""
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the reference arm uses every host core it may run on
    threads = host_threads()
    torch.set_num_threads(threads)
    from tilelang import workloads
    w = workloads.llama8b_memory_ops(tokens=args.tokens)
    total = sum(workloads.llama8b_algorithmic_bytes(tokens=args.tokens).values())
    import oracle.ops as O
    cap_w, cap_s = 3, 30                 # a pass is ~0.2 s on 32 cores: 30 passes keep the arm under a minute
    warmup = max(1, min(args.warmup, cap_w))
    steps = max(1, min(args.steps, cap_s))
    for _ in range(warmup):
        cpu_pass(w, O)
    t = time.perf_counter()
    for _ in range(steps):
        cpu_pass(w, O)
    dt = (time.perf_counter() - t) / steps
    gbs = total / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_for(max(args.gpus, 1), args.tokens),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} full passes of the {args.tokens}-token workload on {threads} threads "
                                   "(torch-CPU restatement of the demos' check functions; the reference's "
                                   "cmodel emulator is not installable); steps above "
                                   f"{cap_s} and warm-up above {cap_w} are capped to bound the run"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
class Step:
    """The four launches of one step over this rank's rows, for one input set."""

    def __init__(self, ops, d, outs, eps):
        self.ops, self.d, self.o, self.eps = ops, d, outs, eps

    def head(self):
        d, o = self.d, self.o
        self.ops.rmsnorm(d["x"], o["y"], d["weight"], eps=self.eps)
        self.ops.rope(d["q"], d["cos"], d["sin"], o["qo"])
        self.ops.rope(d["k"], d["cos"], d["sin"], o["ko"])

    def tail(self):
        self.ops.swiglu(self.d["gate"], self.d["up"], self.o["so"])

    def full(self):
        self.head()
        self.tail()

    def full_concurrent(self, side_streams):
        """The four operators of a step do not depend on one another: issued on four streams (forked from and joined
        to the current one), so that inside a captured graph they are four parallel branches and the three small
        launches run under the SwiGLU launch instead of in front of it."""
        d, o = self.d, self.o
        cur = torch.cuda.current_stream()
        for s in side_streams:
            s.wait_stream(cur)
        with torch.cuda.stream(side_streams[0]):
            self.ops.rmsnorm(d["x"], o["y"], d["weight"], eps=self.eps)
        with torch.cuda.stream(side_streams[1]):
            self.ops.rope(d["q"], d["cos"], d["sin"], o["qo"])
        with torch.cuda.stream(side_streams[2]):
            self.ops.rope(d["k"], d["cos"], d["sin"], o["ko"])
        self.tail()
        for s in side_streams:
            cur.wait_stream(s)


def capture(fn):
    """CUDA graph of the launches `fn` makes (None if this driver/runtime cannot capture them)."""
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g
    except Exception as exc:      # plain launches still measure the kernels; the line says which mode ran
        print(f"bench: graph capture unavailable ({type(exc).__name__}: {exc}); plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS,
                    help="tokens of the batch (default: the named configuration; smaller values are for profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="plain launches instead of CUDA graphs")
    ap.add_argument("--no-kernels", action="store_true",
                    help="skip the per-kernel section (GEMM bf16/FP8, fused MLP, FlashAttention, MLA decode)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    import tilelang
    from tilelang import ops, parallel, workloads
    from tilelang import programs as P

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    # ---- ONE 8192-token problem (seed 1, generated on the CPU so a checker sees the same bits); this rank's rows
    tokens = args.tokens
    w = workloads.llama8b_memory_ops(tokens=tokens, seed=1)
    alg = workloads.llama8b_algorithmic_bytes(tokens=tokens)
    bytes_per_step = sum(alg.values())
    lo, hi = parallel.partition(tokens, world, rank)
    rows = hi - lo
    row_keys = ("x", "q", "k", "cos", "sin", "gate", "up")
    mine = {k: w[k][lo:hi].contiguous() for k in row_keys}
    mine["weight"] = w["weight"]

    # Input sets: set 0 is the problem itself; sets 1.. are the same rows rotated by a few positions (distinct
    # buffers, same values), so that consecutive steps never find their inputs in the 126 MB L2.
    n_sets = max(1, world)
    base = {k: v.to(dev) for k, v in mine.items()}
    sets = [base] + [{k: (torch.roll(v, 7 * s, 0).contiguous() if k in row_keys and k not in ("cos", "sin") else v)
                      for k, v in base.items()} for s in range(1, n_sets)]
    shapes = {"y": (tokens, 4096), "qo": (tokens, 32, 128), "ko": (tokens, 8, 128), "so": (tokens, 14336)}
    gathers = [{k: parallel.ShardedOutput(shp, 0, torch.bfloat16, dev) for k, shp in shapes.items()} for _ in range(n_sets)]
    steps_of = [Step(ops, sets[s], {k: so.local for k, so in gathers[s].items()}, w["eps"]) for s in range(n_sets)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for st in steps_of:                      # warm-up of every set with plain launches (also initialises the library)
        st.full()
    barrier()
    graphs = None
    if not args.no_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        branches = [torch.cuda.Stream(dev) for _ in range(3)]
        concurrent = True
        with torch.cuda.stream(side):
            gs = []
            for st in steps_of:
                full = capture(lambda st=st: st.full_concurrent(branches))
                if full is None:                     # fall back to the four launches in a row
                    concurrent = False
                    full = capture(st.full)
                gs.append((full, capture(st.head), capture(st.tail)))
        torch.cuda.current_stream().wait_stream(side)
        if all(g is not None for trio in gs for g in trio):
            graphs = gs
    if graphs:
        mode = ("CUDA graph replay, the four operators as parallel branches of the graph" if concurrent
                else "CUDA graph replay (4 kernel nodes in a row per step)")
    else:
        mode = "plain launches through the C ABI"

    def run_step(i, ev=None):
        s = i % n_sets
        if ev is None:
            graphs[s][0].replay() if graphs else steps_of[s].full()
            return
        graphs[s][1].replay() if graphs else steps_of[s].head()
        ev[0].record()
        graphs[s][2].replay() if graphs else steps_of[s].tail()
        ev[1].record()

    for i in range(warmup):
        run_step(i)
    barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)

    # events bracket the dominant kernel (SwiGLU, 70% of the bytes) in a quarter of the steps of the timed region
    # (those steps run as two graphs, head then SwiGLU, so that the events see the SwiGLU launch alone)
    n_ev = max(1, min(steps // 4, 64))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ev)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = ops.launch_count()
    if sampler:
        sampler.mark_begin()
    start.record()
    for i in range(steps):
        run_step(i, evs[i // 4] if (i % 4 == 0 and i // 4 < n_ev) else None)
    end.record()
    barrier()
    if sampler:
        sampler.mark_end()
    launches = 4 * steps if graphs else ops.launch_count() - launches0
    ms_total = start.elapsed_time(end)
    swiglu_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    clocks = sampler.stop() if sampler else None

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_per_step = max_over_ranks(ms_total) / steps
    swiglu_ms = max_over_ranks(swiglu_ms)
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- the same steps followed by the all-gather of the four outputs (in place, one NCCL call per output)
    ms_gather = None
    gathered_bytes = sum(2 * int(torch.tensor(shp).prod()) for shp in shapes.values())
    if world > 1:
        g_steps = max(3, min(steps, 50))

        def step_and_gather(i):
            run_step(i)
            for so in gathers[i % n_sets].values():
                so.gather()

        for i in range(3):
            step_and_gather(i)
        barrier()
        s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s1.record()
        for i in range(g_steps):
            step_and_gather(i)
        e1.record()
        barrier()
        ms_gather = max_over_ranks(s1.elapsed_time(e1)) / g_steps
        # the gathered set-0 outputs are the full tensors, in place (rows are the leading dimension)
        assert all(so.full_view() is not None for so in gathers[0].values())

    # ---- end to end: the C2 programs compiled with tilelang.compile, called with pinned host tensors every step
    del sets, steps_of, graphs, base
    gathers = None
    torch.cuda.empty_cache()
    kernels_e2e = {
        "rmsnorm": tilelang.compile(P.rmsnorm(rows, 4096, eps=w["eps"]), out_idx=-1, target="b200"),
        "rope_q": tilelang.compile(P.rope(rows, 32, 128), out_idx=-1, target="b200"),
        "rope_k": tilelang.compile(P.rope(rows, 8, 128), out_idx=-1, target="b200"),
        "swiglu": tilelang.compile(P.swiglu(rows, 14336), out_idx=-1, target="b200"),
    }
    hin = {k: v.pin_memory() for k, v in mine.items()}
    hin["weight"] = hin["weight"].view(1, -1)
    hout = {k: torch.empty((rows,) + shp[1:], dtype=torch.bfloat16).pin_memory() for k, shp in shapes.items()}
    calls = [("rmsnorm", (hin["x"], hin["weight"], hout["y"])), ("rope_q", (hin["q"], hin["cos"], hin["sin"], hout["qo"])),
             ("rope_k", (hin["k"], hin["cos"], hin["sin"], hout["ko"])), ("swiglu", (hin["gate"], hin["up"], hout["so"]))]
    nbytes = lambda t: t.numel() * t.element_size()      # noqa: E731
    h2d = sum(nbytes(t) for _, a in calls for t in a[:-1])
    d2h = sum(nbytes(a[-1]) for _, a in calls)

    def e2e_run(n):
        for _ in range(n):
            for name, a in calls:
                kernels_e2e[name](*a)
        for k in kernels_e2e.values():
            k.adapter.join()

    e2e_steps = max(2, min(steps, 20))
    e2e_run(3)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    e2e_run(e2e_steps)
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2)) / e2e_steps
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9
    h2d_all, d2h_all = max_over_ranks(float(h2d)) * world, max_over_ranks(float(d2h)) * world
    e2e_ok = True
    if rank == 0:                         # what came back is what the device-resident path wrote for the same rows
        import oracle.ops as O
        ref = O.swiglu(mine["gate"][:64], mine["up"][:64])
        e2e_ok = bool(torch.allclose(hout["so"][:64].float(), ref.float(), atol=2e-2, rtol=2e-2))

    del hin, hout, calls, kernels_e2e
    torch.cuda.empty_cache()
    peaks = measured_peaks()
    kernels = None
    if not args.no_kernels:
        import kernel_bench
        kernels = kernel_bench.run_all(dev, rank, world, peaks)

    # every rank is done with the GPU: leave the process group first, so that no rank spins in a collective on the
    # host cores while rank 0 times the CPU baseline
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()

    if rank == 0:
        peak, peak_kind = peaks["hbm_gbs"], peaks["note"].replace("of ", "")
        swiglu_bytes = alg["swiglu"] / world                     # bytes one launch moves on one GPU
        achieved = swiglu_bytes / (swiglu_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_for(world, tokens),
            "launch_mode": mode, "bytes_per_step": bytes_per_step, "rows_per_gpu": rows, "input_sets_per_gpu": n_sets,
            "roofline": {"bound": "hbm", "kernel": "swiglu_kernel", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                         "traffic": SWIGLU_DRAM_BYTES_PER_TOKEN * rows,
                         "traffic_source": "dram__bytes of one ncu capture at 4096 tokens, scaled by the rows of a launch",
                         "avg_launch_ms": swiglu_ms, "bytes_per_launch": swiglu_bytes,
                         "timing": f"CUDA events around the SwiGLU launch in {n_ev} steps of the timed region (every fourth step)"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(h2d_all), "d2h_bytes_per_step": int(d2h_all),
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "path": "tilelang.compile(program, target='b200') JITKernel called with pinned host tensors; "
                            "staging streams and buffers owned by the adapter", "results_checked": e2e_ok},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if ms_gather is not None:
            line["ms_with_output_gather"] = ms_gather
            line["output_gather"] = {"bytes_gathered_per_step": gathered_bytes, "collective": "4 x ncclAllGather, in place",
                                     "ms": ms_gather - ms_per_step,
                                     "gbs_per_gpu_received": gathered_bytes * (world - 1) / world / max((ms_gather - ms_per_step) * 1e-3, 1e-9) / 1e9}
        if kernels is not None:
            line["kernels"] = kernels
        if not args.no_cpu_baseline:
            threads = host_threads()
            torch.set_num_threads(threads)
            cpu_gbs, cpu_s = time_cpu(w, bytes_per_step, reps=2 if world > 1 else 3)
            line["cpu_baseline"] = {
                "value": cpu_gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"best of {2 if world > 1 else 3} full passes of the same {tokens}-token workload ({cpu_s:.2f} s per pass)"}
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
