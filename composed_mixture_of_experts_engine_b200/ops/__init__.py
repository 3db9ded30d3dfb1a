"""Kernels and their autograd wrappers (the reference's ``pkg.kernels`` lives here as ``ops``)."""

from .moe_router import (  # noqa: F401
    TRITON_AVAILABLE,
    MoERouter,
    MoERouterAutograd,
    MoERouterFunction,
    RouterProfile,
    moe_topk_route,
)

__all__ = [
    "MoERouter",
    "MoERouterAutograd",
    "MoERouterFunction",
    "RouterProfile",
    "moe_topk_route",
    "TRITON_AVAILABLE",
]
