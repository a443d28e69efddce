"""Hand-written CUDA kernels for sm_100a and their Python faces."""
from . import build, ops
from .build import KernelBuildError, build_all
from .ops import KernelError

__all__ = ["build", "ops", "KernelBuildError", "KernelError", "build_all"]
