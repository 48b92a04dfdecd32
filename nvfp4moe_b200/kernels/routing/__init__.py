"""Routing kernels: stable dispatch and deterministic combine."""

from .combine import moe_finalize
from .dispatch import MoEDispatch, moe_dispatch

__all__ = ["MoEDispatch", "moe_dispatch", "moe_finalize"]
