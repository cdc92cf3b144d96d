"""Tuner (interface of tilelang/autotuner/__init__.py:90-345 of the reference: `AutoTuner.from_kernel(fn, configs)
.set_compile_args(...).run()` -> `AutotuneResult`).

The reference tunes the block sizes of a program, because its code generator emits exactly the tiling the program
spells out.  Here a matched program runs a library kernel that picks its own decomposition, so two things can be
tuned: (1) any parameter of a program BUILDER (as in the reference - it matters for programs that run on the
tile-op executor, and costs nothing for matched ones), and (2) the tile choices of the library kernels
themselves, per shape, stored in the tile table of `tilelang.cache` where `tilelang.ops` looks them up.
Every candidate is timed on the GPU with CUDA events (`Profiler.do_bench`); nothing here runs without a device.
"""
from __future__ import annotations

import inspect
import itertools
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch


@dataclass(frozen=True)
class AutotuneResult:
    latency: float                # best time per call, ms
    config: dict
    ref_latency: Optional[float]
    libcode: str                  # listing of the best kernel (`get_kernel_source()`)
    func: Any
    kernel: Callable
    trials: List[dict]            # every candidate with its latency (or the reason it was rejected)


def _as_dicts(fn: Callable, configs: Iterable) -> List[dict]:
    names = list(inspect.signature(fn).parameters)
    out = []
    for c in configs:
        out.append(dict(c) if isinstance(c, dict) else dict(zip(names, c)))
    return out


class AutoTuner:
    """Times `tilelang.compile(fn(**config))` for every config and keeps the fastest."""

    def __init__(self, fn: Callable, configs):
        self.fn = fn
        self.configs = _as_dicts(fn, configs)
        self._args: Dict[str, Any] = dict(out_idx=-1, ref_prog=None, supply_prog=None, rtol=1e-2, atol=1e-2,
                                          skip_check=False, target="b200")

    @classmethod
    def from_kernel(cls, kernel: Callable, configs) -> "AutoTuner":
        return cls(kernel, configs)

    def set_compile_args(self, out_idx=-1, supply_type=None, ref_prog: Callable = None, supply_prog: Callable = None,
                         rtol: float = 1e-2, atol: float = 1e-2, max_mismatched_ratio: float = 0.01,
                         skip_check: bool = False, cache_input_tensors: bool = True, target: str = "auto") -> "AutoTuner":
        self._args.update(out_idx=out_idx, ref_prog=ref_prog, supply_prog=supply_prog, rtol=rtol, atol=atol,
                          skip_check=skip_check, target="b200" if target == "auto" else target)
        return self

    def run(self, warmup: int = 5, rep: int = 20, timeout: int = 100) -> AutotuneResult:
        import tilelang
        a = self._args
        best = None
        trials = []
        ref_latency = None
        for cfg in self.configs:
            try:
                func = self.fn(**cfg)
                kernel = tilelang.compile(func, out_idx=a["out_idx"], target=a["target"])
                prof = kernel.get_profiler()
                if a["ref_prog"] is not None and not a["skip_check"]:
                    prof.assert_allclose(a["ref_prog"], rtol=a["rtol"], atol=a["atol"])
                ms = prof.do_bench(warmup=warmup, rep=rep)
            except Exception as exc:           # a config the program cannot take (tiling rule, shapes) is skipped
                trials.append({"config": cfg, "error": f"{type(exc).__name__}: {exc}"})
                continue
            trials.append({"config": cfg, "latency": ms})
            if best is None or ms < best[0]:
                best = (ms, cfg, func, kernel)
        if best is None:
            raise RuntimeError(f"no configuration could be compiled and run: {trials}")
        ms, cfg, func, kernel = best
        return AutotuneResult(latency=ms, config=cfg, ref_latency=ref_latency, libcode=kernel.get_kernel_source(),
                              func=func, kernel=kernel, trials=trials)

    def __call__(self) -> AutotuneResult:
        return self.run()


def autotune(configs: Any, warmup: int = 5, rep: int = 20, timeout: int = 100):
    """Decorator form: `@autotune(configs=[...])` over a program builder; calling the result runs the tuner."""
    def decorator(fn: Callable) -> AutoTuner:
        return AutoTuner(fn, configs)
    return decorator


def product_configs(**axes) -> List[dict]:
    """Cartesian product of named axes, e.g. product_configs(block_M=[32, 64], block_N=[64, 128])."""
    keys = list(axes)
    return [dict(zip(keys, vals)) for vals in itertools.product(*(axes[k] for k in keys))]


# ------------------------------------------------------------------------------- library kernels
def _time_ms(fn: Callable[[], Any], warmup: int, rep: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(rep):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / rep


def tune_gemm(m: int, n: int, k: int, dtype: torch.dtype = torch.bfloat16, transpose_b: bool = False,
              out_dtype: Optional[torch.dtype] = None, warmup: int = 3, rep: int = 10, store: bool = True) -> dict:
    """Measure the C-tile forms of the tensor-core GEMM (64 / 128 / 256 columns on one CTA, 256 x 256 on a CTA pair)
    for one shape and record the fastest in the tile table; `tilelang.ops.gemm` (and every matmul program bound to it) uses it from then on."""
    from .. import ops
    from ..cache import set_tile_choice
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn(m, k, generator=g, device=dev).to(dtype)
    b = torch.randn((n, k) if transpose_b else (k, n), generator=g, device=dev).to(dtype)
    c = torch.empty(m, n, dtype=out_dtype or (torch.bfloat16 if dtype == torch.float8_e4m3fn else dtype), device=dev)
    trials = {}
    for tile_n in (64, 128, 256, 512):            # 512 = 256 x 256 tiles on CTA pairs
        try:
            trials[tile_n] = _time_ms(lambda: ops.gemm(a, b, c, transpose_b, tile_n=tile_n), warmup, rep)
        except RuntimeError as exc:
            trials[tile_n] = str(exc)
    timed = {t: v for t, v in trials.items() if isinstance(v, float)}
    if not timed:
        raise RuntimeError(f"no tile width ran for this shape: {trials}")
    best = min(timed, key=timed.get)
    choice = {"tile_n": best, "ms": timed[best], "trials_ms": {str(t): v for t, v in trials.items()}}
    if store:
        set_tile_choice("gemm", choice, m=m, n=n, k=k, dtype=str(dtype), transpose_b=bool(transpose_b))
    return choice
