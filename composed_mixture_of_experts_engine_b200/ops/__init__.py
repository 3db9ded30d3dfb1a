"""Kernels and their autograd wrappers (the reference's ``pkg.kernels`` lives here as ``ops``).

``moe_router`` carries the public router API of the reference (pkg/kernels/__init__.py); ``functional`` the autograd
ops over the CUDA extension, ``optim`` the fused AdamW, ``attention`` / ``attention_sm100`` causal attention,
``kernels`` the thin launch wrappers and the status word, ``_ext`` the in-tree build.
"""

from .moe_router import MoERouter, MoERouterAutograd, MoERouterFunction, RouterProfile, TRITON_AVAILABLE, moe_topk_route

__all__ = ("MoERouter", "MoERouterAutograd", "MoERouterFunction", "RouterProfile", "TRITON_AVAILABLE", "moe_topk_route")
