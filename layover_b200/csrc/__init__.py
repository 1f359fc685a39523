"""Hand-written CUDA kernels for sm_100a and their loader."""

from .build import ExtensionError, build_all, ensure_built, load

__all__ = ["ExtensionError", "build_all", "ensure_built", "load"]
