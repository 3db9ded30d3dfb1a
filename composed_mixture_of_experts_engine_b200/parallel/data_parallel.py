"""Data parallelism with sharded optimizer state (the role FSDP2 plays in the reference).

``apply_fsdp2(model, topology, mixed_precision_dtype=None)`` keeps the reference's signature and its no-op
cases (dp == 1 or no process groups; pkg/distributed/data_parallel.py:40-98).  What it sets up differs:
the reference wraps modules with ``torch.distributed.fsdp.fully_shard`` (parameter all-gather before use,
gradient reduce-scatter after), whose root wrap also swallows the expert weights although they must only
be reduced across replicas of the same experts.  Here the model keeps whole bf16 parameters resident
(they fit: 180 GB of HBM per GPU) and the *optimizer* shards the fp32 master weights and moments over the
data-parallel group: gradients are reduce-scattered (fp32 accumulation, 1/dp scale), the update runs on the
shard, the bf16 parameters are all-gathered (``ops/optim.py``, ``symm_dp.py``).  Dense parameters use the
dense-replica group (``ddp``: the data-parallel group, times the expert-parallel group when that is a mesh axis of
its own), expert parameters the expert-data-parallel group (``edp``).

This function marks the parameters with their reduction group, makes all replicas start from identical
values, and optionally casts the model to the mixed-precision compute dtype.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .mesh import ParallelTopology, ddp_process_group, edp_process_group

__all__ = ["apply_fsdp2", "mark_expert_params"]


def mark_expert_params(model: nn.Module) -> int:
    """Tag the stacked expert weights of every MoE layer (``is_expert_param``); returns how many were tagged."""
    from .moe_layer import DistributedMoELayer

    n = 0
    for m in model.modules():
        if isinstance(m, DistributedMoELayer):
            for p in (m.w13, m.w2):
                p.is_expert_param = True
                n += 1
    return n


def apply_fsdp2(model: nn.Module, topology: Optional[ParallelTopology],
                mixed_precision_dtype: Optional[torch.dtype] = None) -> nn.Module:
    mark_expert_params(model)
    if mixed_precision_dtype is not None and mixed_precision_dtype != torch.float32:
        model.to(mixed_precision_dtype)
    if (topology is None or topology.mesh is None or not dist.is_initialized()
            or (topology.data_replicas == 1 and topology.axis_size("edp") == 1)):
        return model
    # dense parameters are replicated over every rank that draws its own data: the data-parallel group, and the
    # expert-parallel group too when it is a mesh axis of its own (its ranks exchange tokens, not dense weights)
    dp_group, edp_group = ddp_process_group(topology), edp_process_group(topology)
    dp_src = topology.axis_ranks("ddp")[0]
    edp_src = topology.axis_ranks("edp")[0]
    with torch.no_grad():
        for p in model.parameters():
            if getattr(p, "is_expert_param", False):
                if edp_group is not None:
                    dist.broadcast(p.data, src=edp_src, group=edp_group)
            elif dp_group is not None:
                dist.broadcast(p.data, src=dp_src, group=dp_group)
    model._dp_sharded = True  # type: ignore[attr-defined]
    return model
