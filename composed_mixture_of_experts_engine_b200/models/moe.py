"""The reference's toy language model: Embedding -> N x (RMSNorm + MoE + residual) -> RMSNorm -> Linear.

Module structure and attribute names follow pkg/models/moe.py:63-236 (``embed``, ``blocks[i].norm`` /
``.moe``, ``norm``, ``lm_head``, ``count_parameters``), so checkpoints and telemetry code address the same
paths.  ``ToyMoEBlock`` forwards ``capacity_dropping`` to its layer (the reference dropped that argument,
``moe.py:115-123``).
"""

from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from ..ops import functional as OF
from ..parallel.mesh import ParallelTopology
from ..parallel.moe_layer import DistributedMoELayer
from .registry import register_model

__all__ = ["RMSNorm", "ToyMoEBlock", "ToyMoEModel", "build_model", "DTYPE_MAP"]

DTYPE_MAP = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


class RMSNorm(nn.Module):
    """y = x * rsqrt(mean(x^2) + eps) * weight, computed in fp32 (one kernel on CUDA bf16)."""

    def __init__(self, dim: int, eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return OF.rmsnorm(x, self.weight.to(x.dtype) if self.weight.dtype != x.dtype else self.weight, self.eps)


class ToyMoEBlock(nn.Module):
    def __init__(self, hidden_dim: int, ffn_dim: int, num_experts: int, top_k: int, topology: ParallelTopology,
                 capacity_factor: float = 1.25, dtype: torch.dtype = torch.float32, capacity_dropping: bool = False):
        super().__init__()
        self.norm = RMSNorm(hidden_dim, dtype=dtype)
        self.moe = DistributedMoELayer(hidden_dim=hidden_dim, ffn_dim=ffn_dim, num_experts=num_experts, top_k=top_k,
                                       topology=topology, capacity_factor=capacity_factor,
                                       capacity_dropping=capacity_dropping, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.moe(self.norm(x))


@register_model("toy_moe")
class ToyMoEModel(nn.Module):
    def __init__(self, cfg, topology: ParallelTopology):
        super().__init__()
        m = cfg.model
        dtype = DTYPE_MAP.get(m.dtype, torch.float32)
        self.cfg = cfg
        self.embed = nn.Embedding(m.vocab_size, m.hidden_dim, dtype=dtype)
        self.blocks = nn.ModuleList([
            ToyMoEBlock(m.hidden_dim, m.ffn_dim, m.num_experts, m.top_k, topology, m.capacity_factor, dtype,
                        capacity_dropping=m.capacity_dropping)
            for _ in range(m.num_layers)])
        self.norm = RMSNorm(m.hidden_dim, dtype=dtype)
        self.lm_head = nn.Linear(m.hidden_dim, m.vocab_size, bias=False, dtype=dtype)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.embed(ids)
        for blk in self.blocks:
            x = blk(x)
        return OF.linear(self.norm(x), self.lm_head.weight)

    def moe_layers(self):
        return [blk.moe for blk in self.blocks]

    def aux_losses(self):
        """(mean load-balance loss, mean z-loss) over the MoE layers of the last forward, as tensors."""
        aux = [blk.moe.router.last_aux_loss for blk in self.blocks if blk.moe.router.last_aux_loss is not None]
        z = [blk.moe.router.last_z_loss for blk in self.blocks if blk.moe.router.last_z_loss is not None]
        zero = self.norm.weight.new_zeros((), dtype=torch.float32)
        return (torch.stack(aux).mean() if aux else zero), (torch.stack(z).mean() if z else zero)

    def count_parameters(self) -> Dict[str, int]:
        total = sum(p.numel() for p in self.parameters())
        embed = sum(p.numel() for p in self.embed.parameters()) + sum(p.numel() for p in self.lm_head.parameters())
        router = sum(p.numel() for blk in self.blocks for p in blk.moe.router.parameters())
        experts = sum(blk.moe.w13.numel() + blk.moe.w2.numel() for blk in self.blocks)
        return {"total": total, "embed": embed, "moe_router": router, "moe_experts": experts,
                "other": total - embed - router - experts}


def build_model(cfg, topology: ParallelTopology) -> nn.Module:
    """Build the model named by ``cfg.model.arch`` (default: the toy model) on ``topology.device``."""
    from .registry import build_model_from_config

    return build_model_from_config(cfg, topology)
