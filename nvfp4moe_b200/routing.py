"""Public MoE routing API (``lightmoe/routing.py`` of the reference), plus the router step."""

from .kernels.routing.dispatch import MoEDispatch
from .kernels.routing.router import route_topk

__all__ = ["MoEDispatch", "route_topk"]
