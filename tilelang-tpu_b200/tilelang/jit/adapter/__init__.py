from .base import BaseKernelAdapter  # noqa: F401
from .b200 import B200KernelAdapter  # noqa: F401
