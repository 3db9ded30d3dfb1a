"""Import-path compatibility with the reference package layout.

The reference ships its code as ``pkg`` (``pkg.kernels``, ``pkg.distributed``, ``pkg.models``, ``pkg.elastic``,
``pkg.telemetry``, ``pkg.utils``).  This package maps those paths onto
``composed_mixture_of_experts_engine_b200`` so that code written against the reference imports unchanged:

    from pkg.kernels.moe_router import MoERouter
    from pkg.distributed.parallel_mesh import DistributedMoELayer
    from pkg.elastic.fault_monitor import AsyncCheckpointer
"""

import importlib
import sys

import composed_mixture_of_experts_engine_b200 as _impl

__version__ = _impl.__version__

_MAP = {
    "pkg.kernels": "composed_mixture_of_experts_engine_b200.ops",
    "pkg.kernels.moe_router": "composed_mixture_of_experts_engine_b200.ops.moe_router",
    "pkg.distributed": "composed_mixture_of_experts_engine_b200.parallel",
    "pkg.models": "composed_mixture_of_experts_engine_b200.models",
    "pkg.elastic": "composed_mixture_of_experts_engine_b200.elastic",
    "pkg.elastic.fault_monitor": "composed_mixture_of_experts_engine_b200.elastic.fault_monitor",
    "pkg.telemetry": "composed_mixture_of_experts_engine_b200.telemetry",
    "pkg.telemetry.logger": "composed_mixture_of_experts_engine_b200.telemetry.logger",
    "pkg.utils": "composed_mixture_of_experts_engine_b200.utils",
    "pkg.utils.config": "composed_mixture_of_experts_engine_b200.utils.config",
    "pkg.utils.mfu": "composed_mixture_of_experts_engine_b200.utils.mfu",
    "pkg.models.moe": "composed_mixture_of_experts_engine_b200.models.moe",
    "pkg.models.registry": "composed_mixture_of_experts_engine_b200.models.registry",
}
for _sub in ("mesh", "tensor_parallel", "sequence_parallel", "expert_parallel", "pipeline_parallel", "data_parallel",
             "router", "moe_layer", "parallel_mesh"):
    _MAP[f"pkg.distributed.{_sub}"] = f"composed_mixture_of_experts_engine_b200.parallel.{_sub}"

for _alias, _target in _MAP.items():
    _mod = importlib.import_module(_target)
    sys.modules[_alias] = _mod
    _parent, _, _leaf = _alias.rpartition(".")
    if _parent in sys.modules:
        setattr(sys.modules[_parent], _leaf, _mod) if _parent != "pkg" else None

kernels = sys.modules["pkg.kernels"]
distributed = sys.modules["pkg.distributed"]
models = sys.modules["pkg.models"]
elastic = sys.modules["pkg.elastic"]
telemetry = sys.modules["pkg.telemetry"]
utils = sys.modules["pkg.utils"]
