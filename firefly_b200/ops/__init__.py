from . import kernels
from .build import KernelBuildError
from .kernels import KernelError

__all__ = ["kernels", "KernelBuildError", "KernelError"]
