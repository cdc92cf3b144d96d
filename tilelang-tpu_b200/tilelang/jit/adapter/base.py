"""Adapter base class (interface of tilelang/jit/adapter/base.py:10-57 in the reference)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, List, Optional

from ...engine.param import KernelParam


class BaseKernelAdapter(ABC):
    func: Optional[Callable] = None

    def __init__(self, mod, params: List[KernelParam], result_idx) -> None:
        self.mod = mod
        self.params = params
        self.result_idx = self._legalize_result_idx(result_idx)
        self._post_init()

    def _legalize_result_idx(self, result_idx) -> List[int]:
        n = len(self.params)
        if result_idx is None:
            return []
        if isinstance(result_idx, int):
            if result_idx >= n or result_idx < -n:
                raise ValueError(f"result_idx should be an integer between {-n} and {n - 1}")
            return [result_idx % n]
        if isinstance(result_idx, (list, tuple)):
            out = []
            for idx in result_idx:
                if not isinstance(idx, int) or idx >= n or idx < -n:
                    raise ValueError(f"result_idx should be an integer between {-n} and {n - 1}")
                out.append(idx % n)
            return out
        raise ValueError("result_idx should be a list of integers")

    @abstractmethod
    def _convert_torch_func(self) -> Callable:
        ...

    def __call__(self, *args: Any, **kwds: Any) -> Any:
        return self.func(*args, **kwds)

    def get_kernel_source(self) -> str:
        return self.mod.kernel_source

    def _post_init(self):
        self.func = self._convert_torch_func()
