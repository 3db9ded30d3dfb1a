"""tcgen05 causal attention (forward and backward) for sm_100a: Python side."""

from __future__ import annotations

import torch


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return False


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    raise NotImplementedError
