"""Megatron-style tensor-parallel linears.

``ColumnParallelLinear`` shards the output features (weight ``[out/tp, in]``), ``RowParallelLinear`` the
input features (weight ``[out, in/tp]``).  Signatures follow the reference
(pkg/distributed/tensor_parallel.py:59-212); what differs:

* The column layer gathers its output along the LAST dimension (the reference gathered along dim 0,
  ``tensor_parallel.py:123-130``) and can keep it sharded (``gather_output=False``) so that a
  Column -> elementwise -> Row chain never materialises the full intermediate.
* The row layer accepts either an already sharded input ``[..., in/tp]`` or the full input
  ``[..., in]`` (it then takes its own slice), and reduces with an autograd-aware collective.
* With ``sequence_parallel=True`` the column layer first all-gathers its sequence-sharded input and the
  row layer reduce-scatters its output along the sequence dimension.
* On CUDA with bf16 tensors and a symmetric-memory context the gather / reduce run inside the GEMM
  kernels over NVLink peer memory (``fused_tp``); otherwise the collectives of ``collectives.py`` run.
* The local contraction is ``ops.functional.linear``: the two-SM tcgen05 GEMM on CUDA bf16 tensors (forward,
  input gradient and weight gradient), ``F.linear`` on CPU / fp32.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as OF
from . import collectives as C
from .mesh import ParallelTopology, tp_process_group

__all__ = ["ColumnParallelLinear", "RowParallelLinear"]


def _tp(topology: Optional[ParallelTopology]):
    if topology is None or topology.tp_size == 1:
        return 1, 0, None
    return topology.tp_size, topology.tp_rank, tp_process_group(topology)


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 topology: Optional[ParallelTopology] = None, device=None, dtype=None,
                 gather_output: bool = True, sequence_parallel: bool = False, seq_dim: int = 1):
        super().__init__()
        self.topology = topology
        self.tp_size, self.tp_rank, _ = _tp(topology)
        if out_features % self.tp_size != 0:
            raise ValueError(f"out_features ({out_features}) must be divisible by tp_size ({self.tp_size})")
        self.in_features, self.out_features = in_features, out_features
        self.out_per_rank = out_features // self.tp_size
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel
        self.seq_dim = seq_dim
        self.weight = nn.Parameter(torch.empty(self.out_per_rank, in_features, device=device, dtype=dtype))
        self.weight.tensor_parallel_shard = True  # every tensor-parallel rank holds a different slice
        nn.init.normal_(self.weight, mean=0.0, std=1.0 / math.sqrt(in_features))
        # the bias is kept whole on every rank (as in the reference) and sliced when the output stays sharded
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features} (per rank {self.out_per_rank}), "
                f"tp={self.tp_size}, gather_output={self.gather_output}, sp={self.sequence_parallel}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        group = tp_process_group(self.topology) if self.tp_size > 1 else None
        if self.tp_size > 1:
            if self.sequence_parallel:
                from .fused_tp import allgather_linear

                y = allgather_linear(x, self.weight, self.topology, self.seq_dim)
            else:
                y = OF.linear(C.copy_to_group(x, group), self.weight)
        else:
            y = OF.linear(x, self.weight)
        if self.gather_output and self.tp_size > 1:
            y = C.all_gather(y, y.dim() - 1, group, reduce_scatter_grad=False)
            if self.bias is not None:
                y = y + self.bias
        elif self.bias is not None:
            b = self.bias
            if self.tp_size > 1:
                b = b[self.tp_rank * self.out_per_rank:(self.tp_rank + 1) * self.out_per_rank]
            y = y + b
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 topology: Optional[ParallelTopology] = None, device=None, dtype=None,
                 sequence_parallel: bool = False, seq_dim: int = 1):
        super().__init__()
        self.topology = topology
        self.tp_size, self.tp_rank, _ = _tp(topology)
        if in_features % self.tp_size != 0:
            raise ValueError(f"in_features ({in_features}) must be divisible by tp_size ({self.tp_size})")
        self.in_features, self.out_features = in_features, out_features
        self.in_per_rank = in_features // self.tp_size
        self.sequence_parallel = sequence_parallel
        self.seq_dim = seq_dim
        self.weight = nn.Parameter(torch.empty(out_features, self.in_per_rank, device=device, dtype=dtype))
        self.weight.tensor_parallel_shard = True
        nn.init.normal_(self.weight, mean=0.0, std=1.0 / math.sqrt(in_features))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None

    def extra_repr(self) -> str:
        return (f"in={self.in_features} (per rank {self.in_per_rank}), out={self.out_features}, "
                f"tp={self.tp_size}, sp={self.sequence_parallel}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return OF.linear(x, self.weight, self.bias)
        group = tp_process_group(self.topology)
        if x.shape[-1] == self.in_features and self.in_features != self.in_per_rank:
            x = C.split(x, x.dim() - 1, group)  # full input: take this rank's feature slice
        elif x.shape[-1] != self.in_per_rank:
            raise ValueError(f"RowParallelLinear expects last dim {self.in_per_rank} (sharded) or "
                             f"{self.in_features} (full), got {x.shape[-1]}")
        if self.sequence_parallel:
            from .fused_tp import linear_reduce_scatter

            y = linear_reduce_scatter(x, self.weight, self.topology, self.seq_dim)
        else:
            y = C.all_reduce(OF.linear(x, self.weight), group)
        if self.bias is not None:
            y = y + self.bias
        return y
