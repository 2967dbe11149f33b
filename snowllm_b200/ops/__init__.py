"""Kernel entry points (csrc/*.cu through ctypes) and the shape-to-kernel choice for products."""
from . import kernels  # noqa: F401
from .linear import (grouped_linear, grouped_linear_swiglu, interleave_gate_up, linear,  # noqa: F401
                     linear_swiglu)
