"""Kernel entry points (csrc/*.cu through ctypes) and the shape-to-kernel choice for products."""
from . import kernels  # noqa: F401
from .linear import grouped_linear, linear  # noqa: F401
