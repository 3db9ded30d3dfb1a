"""Parallelism primitives (the reference's ``pkg.distributed``): mesh, TP, SP, EP, PP, DP, router, MoE layer."""

from .data_parallel import apply_fsdp2
from .expert_parallel import all_to_all_combine, all_to_all_dispatch
from .mesh import (ParallelTopology, build_topology, dp_process_group, edp_process_group, ep_process_group,
                   pp_process_group, tp_process_group)
from .moe_layer import DistributedMoELayer, compute_capacity_drop_mask
from .pipeline_parallel import PipelineStage, partition_layers
from .router import MoERouterInterface, RouterStats
from .sequence_parallel import (gather_from_sequence_parallel, reduce_scatter_to_sequence_parallel,
                                scatter_to_sequence_parallel)
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

__all__ = [
    "ParallelTopology", "build_topology", "tp_process_group", "pp_process_group", "ep_process_group",
    "dp_process_group", "edp_process_group", "ColumnParallelLinear", "RowParallelLinear",
    "scatter_to_sequence_parallel", "gather_from_sequence_parallel", "reduce_scatter_to_sequence_parallel",
    "all_to_all_dispatch", "all_to_all_combine", "PipelineStage", "partition_layers", "apply_fsdp2",
    "DistributedMoELayer", "compute_capacity_drop_mask", "MoERouterInterface", "RouterStats",
]
