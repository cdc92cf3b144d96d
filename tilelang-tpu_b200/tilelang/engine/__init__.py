"""Lowering: trace -> match -> bound CUDA program (role of tilelang/engine/lower.py:195-250)."""
from .param import CompiledArtifact, KernelParam  # noqa: F401
from .matcher import BoundKernel, UnsupportedProgram, bind  # noqa: F401
from .lower import lower  # noqa: F401
