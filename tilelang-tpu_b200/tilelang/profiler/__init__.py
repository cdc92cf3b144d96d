"""Measurement helpers (role of tilelang/profiler/__init__.py:22-229 and profiler/bench.py:9-102):
CUDA-event timing with an L2 flush between repetitions, and tensor comparison with a bounded
mismatch ratio."""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..engine.param import KernelParam


def do_bench(fn: Callable, warmup: int = 5, rep: int = 20, flush_l2: bool = True, return_mode: str = "mean") -> float:
    """Milliseconds per call of `fn`, timed with CUDA events on the current stream.  Between
    repetitions a 256 MB buffer is overwritten so inputs do not stay in the 126 MB L2."""
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda") if flush_l2 else None
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rep):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    t = torch.tensor(times)
    return {"mean": t.mean, "median": t.median, "min": t.min, "max": t.max}[return_mode]().item()


def assert_allclose(a: torch.Tensor, b: torch.Tensor, rtol: float = 1e-2, atol: float = 1e-2,
                    max_mismatched_ratio: float = 0.0) -> None:
    """allclose with a tolerated fraction of mismatching elements (tilelang/utils/tensor.py:212-300)."""
    a32, b32 = a.detach().float().cpu(), b.detach().float().cpu()
    bad = (a32 - b32).abs() > atol + rtol * b32.abs()
    ratio = bad.float().mean().item() if bad.numel() else 0.0
    if ratio > max_mismatched_ratio:
        raise AssertionError(f"{int(bad.sum())} of {bad.numel()} elements mismatch (ratio {ratio:.3g} > "
                             f"{max_mismatched_ratio}); max abs diff {(a32 - b32).abs().max().item():.4g}")


class Profiler:
    def __init__(self, params: List[KernelParam], result_idx: List[int], supply_type=None):
        self.params, self.result_idx, self.supply_type = params, result_idx, supply_type
        self.adapter = None

    def with_default_adapter(self, adapter) -> "Profiler":
        self.adapter = adapter
        return self

    def _inputs(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        out = []
        for p in self.params:
            if p.dtype.is_floating_point:
                out.append(torch.randn(*p.shape, generator=g).to(p.dtype).cuda())
            else:
                out.append(torch.zeros(*p.shape, dtype=p.dtype, device="cuda"))
        return out

    def run_once(self, func: Optional[Callable] = None):
        ins = self._inputs()
        return (func or self.adapter)(*ins)

    def assert_allclose(self, reference_program: Callable, atol: float = 1e-2, rtol: float = 1e-2,
                        max_mismatched_ratio: float = 0.01):
        """Run the kernel and `reference_program(*inputs)` (the parameters that are not outputs, in order) and
        compare every output (profiler/__init__.py:76-122)."""
        ins = self._inputs()
        self.adapter(*ins)
        torch.cuda.synchronize()
        ref = reference_program(*[t for i, t in enumerate(ins) if i not in self.result_idx])
        ref = list(ref) if isinstance(ref, (tuple, list)) else [ref]
        if len(ref) != len(self.result_idx):
            raise ValueError(f"the reference returned {len(ref)} tensors for {len(self.result_idx)} outputs")
        for i, r in zip(self.result_idx, ref):
            assert_allclose(ins[i], r, rtol=rtol, atol=atol, max_mismatched_ratio=max_mismatched_ratio)

    def assert_consistent(self, repeat: int = 10):
        """Run-to-run determinism: outputs must be bit-identical (profiler/__init__.py:124-141)."""
        ins = self._inputs()
        self.adapter(*ins)
        ref = [ins[i].clone() for i in self.result_idx]
        for _ in range(repeat):
            self.adapter(*ins)
            for i, r in zip(self.result_idx, ref):
                assert torch.equal(ins[i].view(torch.uint8), r.view(torch.uint8)), "outputs differ between runs"

    def do_bench(self, func: Optional[Callable] = None, warmup: int = 5, rep: int = 20, **_):
        ins = self._inputs()
        f = func or self.adapter
        return do_bench(lambda: f(*ins), warmup=warmup, rep=rep)
