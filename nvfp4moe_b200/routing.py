"""Public MoE routing API (``lightmoe/routing.py`` of the reference)."""

from .kernels.routing.dispatch import MoEDispatch

__all__ = ["MoEDispatch"]
