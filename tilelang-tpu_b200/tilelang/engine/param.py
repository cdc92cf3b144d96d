"""Kernel parameter descriptors (same role and field names as the reference's
tilelang/engine/param.py:14-109)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch

from ..language.ir import Buffer, map_torch_type


@dataclass
class KernelParam:
    dtype: torch.dtype
    shape: List[int]

    @classmethod
    def from_buffer(cls, buffer: Buffer) -> "KernelParam":
        return cls(map_torch_type(buffer.dtype), [int(s) for s in buffer.shape])

    def is_scalar(self) -> bool:
        return len(self.shape) == 0

    def is_unsigned(self) -> bool:
        return str(self.dtype).removeprefix("torch.").startswith("uint")

    def is_float8(self) -> bool:
        return str(self.dtype).removeprefix("torch.").startswith("float8")

    def is_boolean(self) -> bool:
        return str(self.dtype).removeprefix("torch.").startswith("bool")


@dataclass
class CompiledArtifact:
    """Result of `lower()`: the traced program, its parameters, a readable listing, and the
    CUDA program it was bound to (`rt_mod` is a `BoundKernel`)."""
    host_mod: Any
    device_mod: Any
    params: List[KernelParam]
    kernel_source: str
    rt_mod: Optional[Any] = None
