"""Hook for a hand-written tcgen05 attention kernel.  None is built: ``supported`` answers False for every input and
``ops.attention.causal_attention`` runs cuDNN's fused attention through ``scaled_dot_product_attention`` (a library
kernel) on CUDA and the fp32 restatement on CPU.  The reference has no attention operator at all
(pkg/models/moe.py:148-186)."""

from __future__ import annotations

import torch


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return False


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    raise NotImplementedError("no hand-written attention kernel is built; use ops.attention.causal_attention")
