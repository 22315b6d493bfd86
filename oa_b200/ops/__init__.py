"""Kernel-level operations on raw tensors (see `kernels.py`)."""
from . import kernels  # noqa: F401
