"""Python side of the CUDA kernels."""
from .library import KernelError, core, require_cuda
from .linear import linear
from . import kernels

__all__ = ["KernelError", "core", "require_cuda", "linear", "kernels"]
