"""Sequence-parallel linears: all-gather -> GEMM (column) and GEMM -> reduce-scatter (row).

``allgather_linear(x, w, topo, seq_dim)``: ``x`` is this rank's sequence shard ``[.., S/tp, .., in]``; the result
is ``F.linear(all_gather_seq(x), w)`` with the full sequence and this rank's output features.
``linear_reduce_scatter(x, w, topo, seq_dim)``: ``x`` has the full sequence and this rank's input features; the
result is this rank's sequence shard of ``sum_ranks F.linear(x_r, w_r)``.

These replace the reference's gather / all-reduce call sites C4-C7 (pkg/distributed/tensor_parallel.py:128,
201-206; sequence_parallel.py:131,165).  Two implementations with identical semantics:

* library path (any device, gloo or NCCL): the autograd-aware collectives of ``collectives.py``;
* peer-memory path (CUDA, bf16, symmetric memory available): ``symm_tp`` pushes the shards over NVLink and the
  tcgen05 GEMM waits per 128-row tile on arrival flags, so the transfer overlaps the math tile by tile.
"""

from __future__ import annotations

import torch

from ..ops import functional as OF
from . import collectives as C
from .mesh import ParallelTopology, tp_process_group


def _use_peer_path(x: torch.Tensor, w: torch.Tensor, topo: ParallelTopology) -> bool:
    if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        return False
    from . import symm

    return symm.enabled_for(topo, "tp")


def allgather_linear(x: torch.Tensor, w: torch.Tensor, topo: ParallelTopology, seq_dim: int = 1) -> torch.Tensor:
    group = tp_process_group(topo)
    if _use_peer_path(x, w, topo):
        from . import symm_tp

        return symm_tp.allgather_linear(x, w, topo, seq_dim)
    return OF.linear(C.all_gather(x, seq_dim, group, reduce_scatter_grad=True), w)


def linear_reduce_scatter(x: torch.Tensor, w: torch.Tensor, topo: ParallelTopology, seq_dim: int = 1) -> torch.Tensor:
    group = tp_process_group(topo)
    if _use_peer_path(x, w, topo):
        from . import symm_tp

        return symm_tp.linear_reduce_scatter(x, w, topo, seq_dim)
    return C.reduce_scatter(OF.linear(x, w), seq_dim, group)
