"""Typed configs: loading, validation, environment overrides, round trip."""
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from composed_mixture_of_experts_engine_b200.utils.config import ConfigValidationError, MoEConfig, load_config

cfg = MoEConfig.from_yaml(ROOT / "configs" / "olmoe_1b7b.yaml")
print("model:", cfg.model.arch, cfg.model.hidden_dim, "x", cfg.model.num_layers, "| experts", cfg.model.num_experts,
      "top", cfg.model.top_k, "| world", cfg.parallelism.world_size)

try:
    MoEConfig.from_dict({"model": {"top_k": 99, "num_experts": 8}})
except ConfigValidationError as exc:
    print("validation error ->", str(exc).splitlines()[1].strip())

os.environ["MOE_TRAINING__LEARNING_RATE"] = "1e-5"
print("env override lr =", MoEConfig.from_dict({"training": {}}).training.learning_rate)
del os.environ["MOE_TRAINING__LEARNING_RATE"]

with tempfile.TemporaryDirectory() as d:
    cfg.to_yaml(Path(d) / "copy.yaml")
    assert MoEConfig.from_yaml(Path(d) / "copy.yaml").to_dict() == cfg.to_dict()
    print("yaml round trip ok")
legacy = load_config(ROOT / "configs" / "smoke.yaml")
print("legacy access:", legacy.model["hidden_dim"], "typed:", legacy.typed().model.hidden_dim)
