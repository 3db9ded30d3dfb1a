"""Config tree: YAML files load, validators fire, env overrides coerce, YAML round trip, legacy shim.
Mirrors the coverage of the reference's tests/test_config.py."""

import warnings
from pathlib import Path

import pytest

from composed_mixture_of_experts_engine_b200.utils.config import (ConfigValidationError, MoEConfig,
                                                                  _apply_env_overrides, _coerce_env_value,
                                                                  load_config)

pytestmark = pytest.mark.cpu
ROOT = Path(__file__).resolve().parent.parent
CONFIGS = ROOT / "configs"


@pytest.mark.parametrize("name", ["default", "smoke", "large_scale", "olmoe_1b7b", "mixtral_8x7b", "cpu_smoke_ep2",
                                  "smoke_gpu"])
def test_shipped_yaml_loads(name):
    cfg = MoEConfig.from_yaml(CONFIGS / f"{name}.yaml")
    assert cfg.model.top_k <= cfg.model.num_experts
    assert cfg.parallelism.world_size >= 1


def test_reference_default_values():
    cfg = MoEConfig.from_yaml(CONFIGS / "default.yaml")
    assert (cfg.model.hidden_dim, cfg.model.num_layers, cfg.model.num_experts, cfg.model.top_k) == (4096, 32, 64, 2)
    assert cfg.model.ffn_dim == 14336 and cfg.model.vocab_size == 128256 and cfg.model.dtype == "bfloat16"
    assert cfg.parallelism.world_size == 64
    assert cfg.model.arch == "toy_moe"  # the reference architecture stays the default


def test_defaults_without_file():
    cfg = MoEConfig()
    assert cfg.training.warmup_steps == 2000 and cfg.checkpoint.retention == 8


@pytest.mark.parametrize("section,field,value,needle", [
    ("model", "top_k", 128, "top_k"),
    ("model", "hidden_dim", 30, "divisible by 8"),
    ("model", "dtype", "int8", "dtype"),
    ("training", "warmup_steps", 10**9, "warmup_steps"),
    ("checkpoint", "remote_uri", "http://x", "remote_uri"),
    ("elastic", "min_nodes", 10**6, "min_nodes"),
])
def test_validators(section, field, value, needle):
    with pytest.raises(ConfigValidationError) as ei:
        MoEConfig.from_dict({section: {field: value}})
    assert needle in str(ei.value)


def test_missing_file_and_bad_yaml(tmp_path):
    with pytest.raises(FileNotFoundError):
        MoEConfig.from_yaml(tmp_path / "nope.yaml")
    p = tmp_path / "list.yaml"
    p.write_text("- a\n- b\n")
    with pytest.raises(ConfigValidationError):
        MoEConfig.from_yaml(p)


def test_env_overrides(monkeypatch):
    monkeypatch.setenv("MOE_TRAINING__LEARNING_RATE", "1e-5")
    monkeypatch.setenv("MOE_MODEL__HIDDEN_DIM", "1024")
    monkeypatch.setenv("MOE_MODEL__CAPACITY_DROPPING", "true")
    monkeypatch.setenv("MOE_NOSUCH__FIELD", "1")
    cfg = MoEConfig.from_dict({"model": {}, "training": {}})
    assert cfg.training.learning_rate == pytest.approx(1e-5) and isinstance(cfg.training.learning_rate, float)
    assert cfg.model.hidden_dim == 1024 and cfg.model.capacity_dropping is True


def test_coerce():
    assert _coerce_env_value("16") == 16 and _coerce_env_value("1e-5") == 1e-5
    assert _coerce_env_value("false") is False and _coerce_env_value("null") is None
    assert _coerce_env_value("bfloat16") == "bfloat16"
    out = _apply_env_overrides({"model": {"top_k": 2}}, {"MOE_MODEL__TOP_K": "4", "OTHER": "x"})
    assert out["model"]["top_k"] == 4


def test_yaml_round_trip(tmp_path):
    cfg = MoEConfig.from_yaml(CONFIGS / "olmoe_1b7b.yaml")
    cfg.to_yaml(tmp_path / "out.yaml")
    assert MoEConfig.from_yaml(tmp_path / "out.yaml").to_dict() == cfg.to_dict()


def test_legacy_shim_and_raw_warning():
    legacy = load_config(CONFIGS / "smoke.yaml")
    assert legacy.model["hidden_dim"] == 32 and legacy.raw["training"]["max_steps"] == 2
    typed = legacy.typed()
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        _ = typed.raw
    assert any(issubclass(x.category, DeprecationWarning) for x in w)


def test_ep_from_dp_world_size():
    cfg = MoEConfig.from_dict({"parallelism": dict(data_parallel=8, expert_parallel=8, ep_from_dp=True)})
    assert cfg.parallelism.world_size == 8
    with pytest.raises(ConfigValidationError):
        MoEConfig.from_dict({"parallelism": dict(data_parallel=6, expert_parallel=4, ep_from_dp=True)})


def test_gqa_validation():
    cfg = MoEConfig.from_dict({"model": dict(hidden_dim=4096, num_heads=32, num_kv_heads=8)})
    assert cfg.model.resolved_head_dim == 128 and cfg.model.resolved_num_kv_heads == 8
    with pytest.raises(ConfigValidationError):
        MoEConfig.from_dict({"model": dict(hidden_dim=4096, num_heads=32, num_kv_heads=5)})


def test_cli_plan_reports_fit_and_misfit(capsys):
    """``cli.py plan``: exit status 0 with the per-GPU table for a configuration that fits a B200, 1 for one that
    does not (the reference's default dimensions on dp8 x ep8)."""
    from scripts import cli

    assert cli.cmd_plan(str(CONFIGS / "mixtral_8x7b.yaml")) == 0
    out = capsys.readouterr().out
    assert "dp2 x ep2 x tp2 x pp2" in out and "fits" in out
    assert cli.cmd_plan(str(CONFIGS / "default.yaml")) == 1
    assert "DOES NOT FIT" in capsys.readouterr().out


def test_lr_schedule_and_parallelism_refit():
    """``lr_at``: linear warm-up, cosine decay to 10 % (reference train.py:108-113).  ``fit_parallelism``: a
    configured mesh that matches the world is kept, otherwise data parallelism (then expert parallelism) shrinks to
    what the started ranks allow, like the reference's train.py:173-186."""
    import math

    from composed_mixture_of_experts_engine_b200.engine import fit_parallelism, lr_at

    assert lr_at(0, 1.0, 10, 100) == pytest.approx(0.1) and lr_at(9, 1.0, 10, 100) == pytest.approx(1.0)
    assert lr_at(10, 1.0, 10, 100) == pytest.approx(1.0)
    assert lr_at(55, 1.0, 10, 100) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5)))
    assert lr_at(100, 1.0, 10, 100) == pytest.approx(0.1) and lr_at(10_000, 1.0, 10, 100) == pytest.approx(0.1)
    assert lr_at(5, 2.0, 0, 10) == pytest.approx(2.0 * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5))))

    def cfg(**par):
        return MoEConfig.from_dict({"model": {"num_experts": 8}, "parallelism": par})

    mixtral = cfg(data_parallel=2, expert_parallel=2, tensor_parallel=2, pipeline_parallel=2, ep_from_dp=True)
    assert fit_parallelism(mixtral, 8) == (2, 2, 2, 2, True)
    assert fit_parallelism(mixtral, 1) == (1, 1, 1, 1, True)
    assert fit_parallelism(mixtral, 4) == (1, 1, 2, 2, True)          # tp x pp kept, one replica left
    olmoe = cfg(data_parallel=8, expert_parallel=8, ep_from_dp=True)
    assert fit_parallelism(olmoe, 4) == (4, 4, 1, 1, True) and fit_parallelism(olmoe, 2) == (2, 2, 1, 1, True)
    assert fit_parallelism(olmoe, 6) == (6, 2, 1, 1, True)            # ep must divide dp and the expert count
    classic = cfg(data_parallel=2, expert_parallel=4)
    assert fit_parallelism(classic, 8) == (2, 4, 1, 1, False)
    assert fit_parallelism(classic, 4) == (1, 4, 1, 1, False) and fit_parallelism(classic, 2) == (1, 2, 1, 1, False)


def test_mark_expert_params_tags_only_the_stacked_expert_weights():
    from composed_mixture_of_experts_engine_b200.models import build_model
    from composed_mixture_of_experts_engine_b200.parallel import build_topology
    from composed_mixture_of_experts_engine_b200.parallel.data_parallel import apply_fsdp2, mark_expert_params

    c = MoEConfig.from_yaml(CONFIGS / "smoke.yaml")
    topo = build_topology(dp_size=1, ep_size=1, device_type="cpu")
    model = build_model(c, topo)
    assert mark_expert_params(model) == 2 * c.model.num_layers
    tagged = {n for n, p in model.named_parameters() if getattr(p, "is_expert_param", False)}
    assert tagged == {f"blocks.{i}.moe.{w}" for i in range(c.model.num_layers) for w in ("w13", "w2")}
    assert apply_fsdp2(model, topo) is model  # dp == 1: nothing else to set up


def test_validate_config_script_reports_per_file_and_sets_the_exit_status(tmp_path, capsys):
    """`scripts/validate_config.py`: directories expand to their YAML files, a bad file fails only itself, a missing
    path or an empty selection is an error (reference: scripts/validate_config.py)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("validate_config_script", ROOT / "scripts" / "validate_config.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    assert mod.main([str(ROOT / "configs")]) == 0
    out = capsys.readouterr().out
    assert "smoke.yaml" in out and "config(s) valid" in out and "FAIL" not in out

    good = tmp_path / "good.yml"
    good.write_text((ROOT / "configs" / "smoke.yaml").read_text())
    bad = tmp_path / "bad.yaml"
    bad.write_text("model:\n  top_k: 99\n  num_experts: 8\n")
    broken = tmp_path / "broken.yaml"
    broken.write_text("model: [unclosed\n")
    assert mod.main([str(tmp_path)]) == 1
    out = capsys.readouterr().out
    assert out.count("FAIL") == 2 and "good.yml" in out and "1 of 3 config(s) valid, 2 failed" in out

    assert mod.main([str(tmp_path / "nowhere.yaml")]) == 1
    empty = tmp_path / "empty"
    empty.mkdir()
    assert mod.main([str(empty)]) == 1
    assert mod.main([]) == 2
