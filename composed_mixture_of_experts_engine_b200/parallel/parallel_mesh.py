"""Compatibility re-exports: the reference's tests and benchmarks import the parallel layer from one module
(pkg/distributed/parallel_mesh.py:64-78)."""

from .data_parallel import apply_fsdp2
from .expert_parallel import all_to_all_combine, all_to_all_dispatch
from .mesh import ParallelTopology, build_topology, pp_process_group, tp_process_group
from .moe_layer import DistributedMoELayer, _cumcount, _SwiGLUExpert, compute_capacity_drop_mask
from .pipeline_parallel import PipelineStage
from .router import MoERouterInterface, RouterStats
from .sequence_parallel import gather_from_sequence_parallel, scatter_to_sequence_parallel
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

__all__ = [
    "ParallelTopology", "build_topology", "tp_process_group", "pp_process_group", "ColumnParallelLinear",
    "RowParallelLinear", "scatter_to_sequence_parallel", "gather_from_sequence_parallel", "all_to_all_dispatch",
    "all_to_all_combine", "PipelineStage", "apply_fsdp2", "DistributedMoELayer", "_SwiGLUExpert",
    "compute_capacity_drop_mask", "_cumcount", "MoERouterInterface", "RouterStats",
]
