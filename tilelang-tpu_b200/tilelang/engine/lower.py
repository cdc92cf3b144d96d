"""`tilelang.lower(func)`: the reference runs TVM passes and the PPL code generator
(tilelang/engine/lower.py:195-250, phase.py:8-77); here it recognises the program and returns
the binding together with a readable listing of the traced op stream."""
from __future__ import annotations

from ..language.ir import PrimFunc
from ..utils.target import determine_target
from .matcher import bind
from .param import CompiledArtifact, KernelParam


def lower(func_or_mod, target="auto", target_host=None, runtime_only=False, mode="pcie") -> CompiledArtifact:
    if not isinstance(func_or_mod, PrimFunc):
        raise TypeError("lower() expects a program produced by @T.prim_func")
    determine_target(target)
    func = func_or_mod
    if func.name == "main":
        # the reference's code generator rejects a kernel named "main" (codegen_ppl.cc:2194-2196);
        # nothing here depends on the name, so it is only normalised
        func.attrs["global_symbol"] = "main_kernel"
    params = [KernelParam.from_buffer(p) for p in func.params]
    bound = bind(func)
    source = f"// bound to {bound.describe()}\n{func.script()}"
    return CompiledArtifact(host_mod=func, device_mod=func, params=params, kernel_source=source, rt_mod=bound)
