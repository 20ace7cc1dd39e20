"""Native sm_100a kernels and their Python wrappers."""

from .extension import build as build_extension
from .extension import load as load_extension

__all__ = ["build_extension", "load_extension"]
