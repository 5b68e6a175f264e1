from . import ops
from .build import KernelBuildError, compile_family, load_family
from .ops import KernelError

__all__ = ["ops", "KernelBuildError", "KernelError", "compile_family", "load_family"]
