"""Names the reference exposes from ``lightmoe/kernels/grouped/kernel.py``."""

from .runtime import DECODE_GRID_DOUBLE, DECODE_GRID_PERSISTENT

__all__ = ["DECODE_GRID_DOUBLE", "DECODE_GRID_PERSISTENT"]
