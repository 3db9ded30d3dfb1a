"""Typed, validated configuration tree for the engine.

Same schema and behaviour as the reference's ``pkg/utils/config.py:94-457`` (six sections,
``MOE_<SECTION>__<KEY>`` environment overrides, YAML round trip, legacy ``load_config`` shim), with
optional additions that default to the reference behaviour:

* ``model.arch / num_heads / num_kv_heads / head_dim / rope_theta / aux_loss_coeff / norm_eps`` –
  the attention + RoPE decoder (``arch: moe_decoder``) that the reference's toy model lacks.
* ``parallelism.ep_from_dp`` – the expert-parallel group is a sub-axis of the data-parallel group
  (world = dp * tp * pp) instead of a separate mesh axis (world = dp * ep * tp * pp).
* ``parallelism.sequence_parallel / pipeline_microbatches``, ``training.seed``,
  ``training.activation_recompute``.
"""

from __future__ import annotations

import copy
import os
import warnings
from pathlib import Path
from typing import Any, Dict, Optional

import yaml
from pydantic import BaseModel, Field, ValidationError, field_validator, model_validator

__all__ = [
    "MoEConfig",
    "ModelConfig",
    "TrainingConfig",
    "ParallelismConfig",
    "CheckpointConfig",
    "ElasticConfig",
    "TelemetryConfig",
    "ConfigValidationError",
    "load_config",
]

_HAS_PYDANTIC = True
_VALID_DTYPES = ("float32", "bfloat16", "float16")


class ConfigValidationError(ValueError):
    """A config source failed validation; the message names every offending field."""


class ModelConfig(BaseModel):
    hidden_dim: int = Field(4096, description="Model width H.")
    num_layers: int = Field(32, description="Number of decoder blocks.")
    num_experts: int = Field(64, description="Experts per MoE layer (E).")
    top_k: int = Field(2, description="Experts evaluated per token (K).")
    capacity_factor: float = Field(1.25, description="Per-expert capacity = ceil(cf * N * K / E).")
    capacity_dropping: bool = Field(False, description="Drop (token, slot) pairs beyond the expert capacity.")
    ffn_dim: int = Field(14336, description="Expert SwiGLU intermediate width (F).")
    vocab_size: int = Field(128256)
    sequence_length: int = Field(4096)
    dtype: str = Field("bfloat16")
    # --- additions (the reference model has no attention) ---
    arch: str = Field("toy_moe", description="Registered model name: toy_moe | moe_decoder.")
    num_heads: int = Field(0, description="Attention heads (0: hidden_dim // 128, at least 1).")
    num_kv_heads: int = Field(0, description="KV heads for grouped-query attention (0: same as num_heads).")
    head_dim: int = Field(0, description="Per-head width (0: hidden_dim // num_heads).")
    rope_theta: float = Field(10000.0)
    aux_loss_coeff: float = Field(0.0, description="Weight of the load-balance loss E * sum_i f_i P_i.")
    norm_eps: float = Field(1e-5)
    init_std: float = Field(0.0, description="Std of the normal init of all matrices (0: each module's default).")

    @model_validator(mode="after")
    def _check(self) -> "ModelConfig":
        if self.top_k > self.num_experts:
            raise ValueError(f"top_k ({self.top_k}) must be <= num_experts ({self.num_experts})")
        if self.top_k < 1:
            raise ValueError("top_k must be >= 1")
        if self.hidden_dim % 8 != 0:
            raise ValueError(f"hidden_dim ({self.hidden_dim}) must be divisible by 8")
        if self.dtype not in _VALID_DTYPES:
            raise ValueError(f"dtype must be one of {set(_VALID_DTYPES)}, got {self.dtype!r}")
        heads = self.resolved_num_heads
        kv = self.num_kv_heads or heads
        if heads % kv != 0:
            raise ValueError(f"num_heads ({heads}) must be a multiple of num_kv_heads ({kv})")
        return self

    @property
    def resolved_num_heads(self) -> int:
        return self.num_heads if self.num_heads > 0 else max(1, self.hidden_dim // 128)

    @property
    def resolved_num_kv_heads(self) -> int:
        return self.num_kv_heads if self.num_kv_heads > 0 else self.resolved_num_heads

    @property
    def resolved_head_dim(self) -> int:
        return self.head_dim if self.head_dim > 0 else self.hidden_dim // self.resolved_num_heads


class TrainingConfig(BaseModel):
    global_batch_size: int = Field(4096)
    micro_batch_size: int = Field(4)
    learning_rate: float = Field(3e-4)
    weight_decay: float = Field(0.1)
    grad_clip: float = Field(1.0)
    max_steps: int = Field(100_000)
    log_interval: int = Field(10)
    ckpt_interval: int = Field(500)
    warmup_steps: int = Field(2000)
    gradient_accumulation_steps: int = Field(4)
    z_loss_weight: float = Field(0.0, description="Router z-loss weight (0 disables).")
    # --- additions ---
    seed: int = Field(0)
    activation_recompute: bool = Field(False)

    @model_validator(mode="after")
    def _check(self) -> "TrainingConfig":
        if self.warmup_steps >= self.max_steps:
            raise ValueError(f"warmup_steps ({self.warmup_steps}) must be < max_steps ({self.max_steps})")
        return self


class ParallelismConfig(BaseModel):
    data_parallel: int = Field(8)
    expert_parallel: int = Field(8)
    tensor_parallel: int = Field(1)
    pipeline_parallel: int = Field(1)
    # --- additions ---
    ep_from_dp: bool = Field(False, description="EP ranks are a sub-axis of DP (world = dp * tp * pp).")
    sequence_parallel: bool = Field(False, description="Megatron sequence parallelism inside TP regions.")
    pipeline_microbatches: int = Field(0, description="Microbatches per 1F1B step (0: gradient_accumulation_steps).")

    @property
    def world_size(self) -> int:
        base = self.data_parallel * self.tensor_parallel * self.pipeline_parallel
        return base if self.ep_from_dp else base * self.expert_parallel

    @model_validator(mode="after")
    def _check(self) -> "ParallelismConfig":
        for name in ("data_parallel", "expert_parallel", "tensor_parallel", "pipeline_parallel"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        if self.ep_from_dp and self.data_parallel % self.expert_parallel != 0:
            raise ValueError(
                f"ep_from_dp needs data_parallel ({self.data_parallel}) divisible by expert_parallel "
                f"({self.expert_parallel})"
            )
        return self


class CheckpointConfig(BaseModel):
    local_dir: str = Field("/mnt/nvme/moe-engine/ckpts")
    remote_uri: str = Field("s3://moe-engine-ckpts/run-001/")
    async_workers: int = Field(4)
    retention: int = Field(8)

    @field_validator("remote_uri")
    @classmethod
    def _uri(cls, v: str) -> str:
        if not (v.startswith("s3://") or v.startswith("file://")):
            raise ValueError(f"remote_uri must start with 's3://' or 'file://', got: {v!r}")
        return v


class ElasticConfig(BaseModel):
    min_nodes: int = Field(8)
    max_nodes: int = Field(256)
    rdzv_backend: str = Field("c10d")
    rdzv_endpoint: str = Field("etcd-headless:2379")
    health_check_interval_s: float = Field(5.0)
    drop_grace_period_s: float = Field(30.0)

    @model_validator(mode="after")
    def _check(self) -> "ElasticConfig":
        if self.min_nodes > self.max_nodes:
            raise ValueError(f"min_nodes ({self.min_nodes}) must be <= max_nodes ({self.max_nodes})")
        return self


class TelemetryConfig(BaseModel):
    log_dir: str = Field("/var/log/moe-engine")
    tensorboard_dir: str = Field("/var/log/moe-engine/tb")
    json_path: str = Field("/var/log/moe-engine/step.jsonl")
    mfu_target: float = Field(0.55)
    hardware_peak_tflops: float = Field(989.0, description="Per-GPU dense bf16 peak used as the MFU denominator.")


class MoEConfig(BaseModel):
    """Root config.  Build with :meth:`from_yaml` / :meth:`from_dict`."""

    model: ModelConfig = Field(default_factory=ModelConfig)
    training: TrainingConfig = Field(default_factory=TrainingConfig)
    parallelism: ParallelismConfig = Field(default_factory=ParallelismConfig)
    checkpoint: CheckpointConfig = Field(default_factory=CheckpointConfig)
    elastic: ElasticConfig = Field(default_factory=ElasticConfig)
    telemetry: TelemetryConfig = Field(default_factory=TelemetryConfig)

    @classmethod
    def from_yaml(cls, path: "str | Path") -> "MoEConfig":
        p = Path(path)
        if not p.exists():
            raise FileNotFoundError(f"Config file not found: {p.resolve()}")
        with p.open("r") as fh:
            raw = yaml.safe_load(fh)
        if not isinstance(raw, dict):
            raise ConfigValidationError(
                f"Config file {p} did not parse to a dict (got {type(raw).__name__}); is the YAML valid?"
            )
        return cls.from_dict(raw, source=str(p))

    @classmethod
    def from_dict(cls, d: Dict[str, Any], source: str = "<dict>") -> "MoEConfig":
        d = _apply_env_overrides(d)
        try:
            return cls(**d)
        except ValidationError as exc:
            lines = [f"Config validation failed (source: {source}):"]
            for err in exc.errors():
                loc = " -> ".join(str(x) for x in err["loc"])
                lines.append(f"  [{loc}]  {err['msg']}")
                if "input" in err:
                    lines.append(f"    got: {err['input']!r}")
            raise ConfigValidationError("\n".join(lines)) from exc
        except (TypeError, KeyError) as exc:
            raise ConfigValidationError(f"Unexpected error loading config from {source}: {exc}") from exc

    def to_dict(self) -> Dict[str, Any]:
        return self.model_dump()

    def to_yaml(self, path: "str | Path") -> None:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with p.open("w") as fh:
            yaml.safe_dump(self.to_dict(), fh, default_flow_style=False, sort_keys=False)

    @property
    def raw(self) -> Dict[str, Any]:
        warnings.warn(
            "MoEConfig.raw is deprecated; access fields directly: cfg.model.hidden_dim",
            DeprecationWarning,
            stacklevel=2,
        )
        return self.to_dict()


class _LegacyConfig:
    """Dict-per-section view kept for callers of the old ``load_config`` API."""

    def __init__(self, cfg: MoEConfig):
        self._cfg = cfg
        d = cfg.to_dict()
        self.model = d["model"]
        self.training = d["training"]
        self.parallelism = d["parallelism"]
        self.checkpoint = d["checkpoint"]
        self.elastic = d["elastic"]
        self.telemetry = d["telemetry"]
        self.raw = d

    def typed(self) -> MoEConfig:
        return self._cfg


def load_config(path: "str | Path") -> _LegacyConfig:
    return _LegacyConfig(MoEConfig.from_yaml(path))


def _coerce_env_value(val: str) -> Any:
    """int, then float (so that ``1e-5`` is a float, which YAML 1.1 would read as a string), then YAML."""
    for caster in (int, float):
        try:
            return caster(val)
        except ValueError:
            continue
    return yaml.safe_load(val)


def _apply_env_overrides(d: Dict[str, Any], environ: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
    """``MOE_TRAINING__LEARNING_RATE=1e-4`` overrides ``d["training"]["learning_rate"]``."""
    env = os.environ if environ is None else environ
    out = copy.deepcopy(d)
    for key, val in env.items():
        if not key.startswith("MOE_"):
            continue
        rest = key[4:].lower()
        section, sep, field_name = rest.partition("__")
        if not sep or section not in out or not isinstance(out[section], dict):
            continue
        out[section][field_name] = _coerce_env_value(val)
    return out
