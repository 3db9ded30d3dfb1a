"""Validating wrapper around the kernel router, with a ``RouterStats`` result.

Follows the reference's ``pkg/distributed/router.py:46-243``: 2-D input only, hidden-size check, token
conservation as a ``RuntimeError``, ``capacity_budget(n) = ceil(cf * n * K / E)`` and a warning when the
capacity factor is below 1.  Reading the statistics costs one device round trip here; the hot path of
``DistributedMoELayer`` therefore calls the kernel router directly and never builds a ``RouterStats``.
"""

from __future__ import annotations

import logging
import math
import warnings
from dataclasses import dataclass

import torch
import torch.nn as nn

log = logging.getLogger(__name__)

__all__ = ["MoERouterInterface", "RouterStats"]


@dataclass
class RouterStats:
    expert_indices: torch.Tensor      # [N, K] int64
    combine_weights: torch.Tensor     # [N, K] token dtype, rows sum to 1
    dispatch_counts: torch.Tensor     # [E] int64
    load_imbalance: float             # max / mean tokens per expert
    router_z_loss: float              # mean(logsumexp(logits)^2)
    used_triton: bool                 # always False here (no Triton path)
    kernel_ms: float
    tokens_per_expert_mean: float
    tokens_per_expert_std: float


class MoERouterInterface(nn.Module):
    def __init__(self, hidden_dim: int, num_experts: int, top_k: int, capacity_factor: float = 1.25,
                 dtype: torch.dtype = torch.float32):
        super().__init__()
        if hidden_dim <= 0 or num_experts <= 0:
            raise ValueError("hidden_dim and num_experts must be positive")
        if not (1 <= top_k <= num_experts):
            raise ValueError(f"top_k ({top_k}) must be in [1, num_experts={num_experts}]")
        if capacity_factor <= 0:
            raise ValueError("capacity_factor must be positive")
        if capacity_factor < 1.0:
            warnings.warn(
                f"capacity_factor={capacity_factor} < 1.0 will silently drop tokens even under perfect balance; "
                "consider a value of at least 1.0", UserWarning, stacklevel=2)
        self.hidden_dim, self.num_experts, self.top_k = hidden_dim, num_experts, top_k
        self.capacity_factor = capacity_factor
        from ..ops.moe_router import MoERouter

        self._kernel_router = MoERouter(hidden_dim=hidden_dim, num_experts=num_experts, top_k=top_k, dtype=dtype)
        self._kernel_router.profile_timing = True

    def extra_repr(self) -> str:
        return (f"hidden_dim={self.hidden_dim}, num_experts={self.num_experts}, top_k={self.top_k}, "
                f"capacity_factor={self.capacity_factor}")

    def forward(self, tokens: torch.Tensor) -> RouterStats:
        if tokens.dim() != 2:
            raise ValueError(
                f"MoERouterInterface.forward expects 2D input [N, H], got shape {list(tokens.shape)}. "
                "Flatten [B, S, H] → [B*S, H] before calling.")
        N, H = tokens.shape
        if H != self.hidden_dim:
            raise ValueError(f"Token hidden dim {H} ≠ router hidden_dim {self.hidden_dim}.")
        idx, weights, counts = self._kernel_router(tokens)
        total = int(counts.sum().item())
        if total != N * self.top_k:
            raise RuntimeError(
                f"Token conservation violation: dispatched {total} tokens but expected {N * self.top_k} "
                f"(N={N}, K={self.top_k}).")
        prof = self._kernel_router.last_profile
        cf = counts.float()
        return RouterStats(
            expert_indices=idx,
            combine_weights=weights,
            dispatch_counts=counts,
            load_imbalance=prof.expert_load_imbalance if prof else 1.0,
            router_z_loss=prof.router_z_loss if prof else 0.0,
            used_triton=False,
            kernel_ms=prof.kernel_ms if prof else 0.0,
            tokens_per_expert_mean=float(cf.mean().item()),
            tokens_per_expert_std=float(cf.std().item()) if self.num_experts > 1 else 0.0,
        )

    def capacity_budget(self, num_tokens: int) -> int:
        return math.ceil(self.capacity_factor * num_tokens * self.top_k / self.num_experts)
