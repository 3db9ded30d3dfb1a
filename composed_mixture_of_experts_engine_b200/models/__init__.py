"""Models and the model registry."""

from .registry import (ModelRegistry, _register_builtins, build_model_from_config, list_registered_models,
                       register_model)

_register_builtins()

from .decoder import MoEDecoder  # noqa: E402
from .moe import RMSNorm, ToyMoEBlock, ToyMoEModel, build_model  # noqa: E402

__all__ = [
    "RMSNorm", "ToyMoEBlock", "ToyMoEModel", "MoEDecoder", "build_model", "register_model",
    "build_model_from_config", "list_registered_models", "ModelRegistry",
]
