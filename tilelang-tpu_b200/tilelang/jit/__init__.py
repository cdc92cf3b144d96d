"""`tilelang.compile` / `tilelang.jit` (signatures of tilelang/jit/__init__.py:24-134)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Union

from ..cache import cached
from ..language.ir import PrimFunc
from .kernel import JITKernel  # noqa: F401


def compile(func: PrimFunc = None, out_idx: Union[List[int], int, None] = None,     # noqa: A001
            execution_backend: str = "cython", target: str = "auto", target_host=None, verbose: bool = False,
            pass_configs: Optional[Dict[str, Any]] = None, mode: str = "pcie") -> JITKernel:
    """Bind a traced program to its CUDA kernels and return a callable JITKernel."""
    return cached(func=func, out_idx=out_idx, execution_backend=execution_backend, target=target,
                  target_host=target_host, verbose=verbose, pass_configs=pass_configs, mode=mode)


def jit(func: Callable = None, *, out_idx: Union[List[int], int, None] = None, execution_backend: str = "cython",
        target: str = "auto", verbose: bool = False, **pass_config_kwargs):
    """Decorator form: `@tilelang.jit(out_idx=-1)` over a function that RETURNS a prim_func; the
    decorated function compiles on call."""

    def wrap(builder: Callable):
        def compiled(*args, **kwargs):
            program = builder(*args, **kwargs)
            return compile(program, out_idx=out_idx, execution_backend=execution_backend, target=target,
                           verbose=verbose, pass_configs=pass_config_kwargs or None)
        compiled.__name__ = getattr(builder, "__name__", "jit_kernel")
        return compiled

    if isinstance(func, PrimFunc):
        return compile(func, out_idx=out_idx, execution_backend=execution_backend, target=target, verbose=verbose)
    return wrap(func) if func is not None else wrap
