"""B200-native implementation of the TileLang-TPU operator path.

Same user surface as the reference (`import tilelang; import tilelang.language as T;
tilelang.compile(func, out_idx=..., target=...)`, cf. tilelang/__init__.py and
tilelang/jit/__init__.py:112-134 there), backed by a pre-built library of hand-written sm_100a
CUDA kernels instead of TVM lowering plus the SOPHGO code generator.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401
from . import ops  # noqa: F401
from . import language  # noqa: F401,E402
from . import programs  # noqa: F401,E402
from .engine import lower  # noqa: F401,E402
from .jit import JITKernel, compile, jit  # noqa: F401,E402
from .cache import cached, clear_cache  # noqa: F401,E402
from .profiler import Profiler  # noqa: F401,E402
from . import autotuner  # noqa: F401,E402
