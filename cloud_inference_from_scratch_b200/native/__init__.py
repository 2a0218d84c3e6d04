from .build import NativeBuildError, build_only, load_library
from .ops import KernelError, Ops

__all__ = ["KernelError", "NativeBuildError", "Ops", "build_only", "load_library"]
