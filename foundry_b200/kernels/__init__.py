"""The CUDA kernel library: build, load, and the checked Python faces."""
from . import library, ops
from .library import KernelLibraryError, build
from .ops import KernelError

__all__ = ["library", "ops", "KernelLibraryError", "build", "KernelError"]
