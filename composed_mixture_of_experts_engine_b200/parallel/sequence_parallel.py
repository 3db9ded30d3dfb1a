"""Megatron sequence parallelism helpers tied to the tensor-parallel group.

``scatter_to_sequence_parallel(x, topo, next_weight=None)`` keeps this rank's ``S/tp`` slice of ``[B, S, H]``
(no communication forward, all-gather backward); ``gather_from_sequence_parallel`` is the inverse
(all-gather forward).  Same names and argument order as the reference
(pkg/distributed/sequence_parallel.py:56-166).

``next_weight``: the fused variant distributes the projection that follows over the group.  Every rank projects
its own ``S/tp`` rows with ``next_weight`` and the results are all-gathered along the sequence, so every rank
returns ``F.linear(x, next_weight)`` of the full sequence, ``[B, S, F]``, having computed ``1/tp`` of it.  This is
the behaviour the reference documents and tests (tests/test_sequence_parallel_v03.py:139-196); its own fused
variant all-reduced different sequence chunks (pkg/distributed/sequence_parallel.py:129-134), which is not that
function.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import functional as OF
from . import collectives as C
from .mesh import ParallelTopology, tp_process_group

__all__ = ["scatter_to_sequence_parallel", "gather_from_sequence_parallel", "reduce_scatter_to_sequence_parallel"]


def _check(x: torch.Tensor, topo: ParallelTopology, seq_dim: int) -> None:
    if x.dim() <= seq_dim:
        raise ValueError(f"expected a tensor with a sequence dimension {seq_dim}, got shape {list(x.shape)}")


def scatter_to_sequence_parallel(x: torch.Tensor, topology: Optional[ParallelTopology],
                                 next_weight: Optional[torch.Tensor] = None, seq_dim: int = 1) -> torch.Tensor:
    tp = 1 if topology is None else topology.tp_size
    if tp > 1:
        _check(x, topology, seq_dim)
        S = x.shape[seq_dim]
        if S % tp != 0:
            raise ValueError(f"sequence length ({S}) must be divisible by tp_size ({tp}) for sequence parallelism")
        x = C.split(x, seq_dim, tp_process_group(topology))
    if next_weight is not None:
        x = OF.linear(x, next_weight)
        if tp > 1:
            # every rank holds the same full-sequence gradient afterwards: the backward keeps this rank's slice
            x = C.all_gather(x, seq_dim, tp_process_group(topology), reduce_scatter_grad=False)
    return x


def gather_from_sequence_parallel(x: torch.Tensor, topology: Optional[ParallelTopology], seq_dim: int = 1,
                                  reduce_scatter_grad: bool = False) -> torch.Tensor:
    """All-gather the sequence shards.  ``reduce_scatter_grad=True`` when the consumer is tensor-parallel
    (every rank then holds a partial gradient of the whole sequence)."""
    if topology is None or topology.tp_size == 1:
        return x
    _check(x, topology, seq_dim)
    return C.all_gather(x, seq_dim, tp_process_group(topology), reduce_scatter_grad=reduce_scatter_grad)


def reduce_scatter_to_sequence_parallel(x: torch.Tensor, topology: Optional[ParallelTopology], seq_dim: int = 1
                                        ) -> torch.Tensor:
    """Sum partial results over the tensor-parallel group and keep this rank's sequence slice."""
    if topology is None or topology.tp_size == 1:
        return x
    return C.reduce_scatter(x, seq_dim, tp_process_group(topology))
