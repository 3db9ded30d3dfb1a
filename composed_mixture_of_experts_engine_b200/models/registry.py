"""Name -> model class registry (``register_model``, ``build_model_from_config``, ``list_registered_models``).

Same behaviour as the reference's ``pkg/models/registry.py:69-209``: duplicate names raise ``ValueError`` naming
the class that already holds the name, unknown names raise ``KeyError`` listing what is registered, built
models are moved to ``topology.device``.  The architecture is read from ``cfg.model.arch`` (a real config field
here; default ``"toy_moe"``).
"""

from __future__ import annotations

import logging
from typing import Callable, Dict, Optional, Type

import torch.nn as nn

__all__ = ["register_model", "build_model_from_config", "list_registered_models", "ModelRegistry"]

log = logging.getLogger(__name__)
_REGISTRY: Dict[str, Type[nn.Module]] = {}


class ModelRegistry:
    @staticmethod
    def register(name: str, cls: Type[nn.Module]) -> None:
        if name in _REGISTRY:
            raise ValueError(
                f"Model '{name}' is already registered as {_REGISTRY[name].__qualname__}. "
                "Use a unique name or remove the existing registration first.")
        _REGISTRY[name] = cls

    @staticmethod
    def get(name: str) -> Type[nn.Module]:
        if name not in _REGISTRY:
            known = ", ".join(f"'{k}'" for k in sorted(_REGISTRY))
            raise KeyError(f"No model registered under name '{name}'. Available: [{known}]. "
                           "Register your model with @register_model('name') before building.")
        return _REGISTRY[name]

    @staticmethod
    def list() -> "list[str]":
        return sorted(_REGISTRY)

    @staticmethod
    def unregister(name: str) -> None:
        _REGISTRY.pop(name, None)


def register_model(name: str) -> Callable[[Type[nn.Module]], Type[nn.Module]]:
    def deco(cls: Type[nn.Module]) -> Type[nn.Module]:
        ModelRegistry.register(name, cls)
        return cls

    return deco


def build_model_from_config(cfg, topology, arch: Optional[str] = None) -> nn.Module:
    if arch is None:
        arch = getattr(cfg.model, "arch", "toy_moe")
    cls = ModelRegistry.get(arch)
    log.info("Building model '%s' (%s) on %s", arch, cls.__qualname__, topology.device)
    import torch

    with torch.device(topology.device):  # parameters are created (and initialised) on the target device
        model = cls(cfg, topology)
    return model.to(topology.device)


def list_registered_models() -> "list[str]":
    return ModelRegistry.list()


def _register_builtins() -> None:
    from . import decoder as _decoder  # noqa: F401
    from . import moe as _moe  # noqa: F401
