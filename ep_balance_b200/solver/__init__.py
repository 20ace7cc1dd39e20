from .api import solve, validate_inputs
from .bisect import solve_bisect
from .device_semantics import solve_device_semantics
from .exact import solve_exact

__all__ = ["solve", "solve_exact", "solve_bisect", "solve_device_semantics", "validate_inputs"]
