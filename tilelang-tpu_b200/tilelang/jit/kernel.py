"""JITKernel (interface of tilelang/jit/kernel.py:21-387 in the reference)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

from ..engine import lower
from ..engine.param import CompiledArtifact, KernelParam
from ..language.ir import PrimFunc
from ..utils.target import determine_target
from .adapter import B200KernelAdapter


class JITKernel:
    """A compiled program: call it with all parameters (outputs are written in place)."""

    def __init__(self, func: PrimFunc = None, out_idx: Union[List[int], int, None] = None,
                 execution_backend: str = "cython", target: str = "auto", target_host=None, verbose: bool = False,
                 pass_configs: Optional[Dict[str, Any]] = None, mode: str = "pcie"):
        # `mode` selected the BM1690 board ("pcie") or its CPU emulator ("cmodel") in the reference
        # (jit/kernel.py:101-104); both spellings are accepted and mean the GPU here.
        assert mode in ("pcie", "cmodel", "b200"), f"Invalid mode: {mode}"
        assert execution_backend in ("dlpack", "ctypes", "cython", "b200"), f"Invalid execution backend {execution_backend}"
        self.prim_func = func
        self.out_idx = out_idx
        self.execution_backend = "b200"
        self.target = determine_target(target)
        self.target_host = target_host
        self.verbose = verbose
        self.pass_configs = pass_configs or {}
        self.mode = mode
        self.artifact: CompiledArtifact = lower(func, target=self.target, mode=mode)
        self.adapter = B200KernelAdapter(self.artifact, self.artifact.params, out_idx, verbose=verbose)
        self.torch_function = self.adapter.func
        if verbose:
            print(self.artifact.kernel_source)

    def __call__(self, *args: Any, **kwds: Any) -> Any:
        return self.torch_function(*args, **kwds)

    @property
    def params(self) -> List[KernelParam]:
        return self.artifact.params

    def get_kernel_source(self) -> str:
        return self.artifact.kernel_source

    def get_host_source(self) -> str:
        return f"// {self.adapter.bound.entry_point} of libtl_b200.so (pre-built; include/tl_b200.h)"

    def get_profiler(self, tensor_supply_type=None):
        from ..profiler import Profiler
        return Profiler(self.params, self.adapter.result_idx, tensor_supply_type).with_default_adapter(self.adapter)

    def run_once(self, func=None) -> None:
        return self.get_profiler().run_once(func)
