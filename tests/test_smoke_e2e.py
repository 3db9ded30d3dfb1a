"""End-to-end: ``train.main`` in-process with a generated YAML; JSONL envelope; both checkpoint tiers populated;
resume from the newest checkpoint (reference: tests/test_smoke_e2e.py, file:// second tier)."""

import json
from pathlib import Path

import pytest
import yaml

pytestmark = pytest.mark.cpu


def _write_cfg(tmp_path: Path, arch: str, max_steps: int) -> Path:
    cfg = {
        "model": dict(hidden_dim=32, num_layers=2, num_experts=4, top_k=2, ffn_dim=64, vocab_size=128,
                      sequence_length=8, dtype="float32", arch=arch, num_heads=2, aux_loss_coeff=0.01),
        "training": dict(global_batch_size=4, micro_batch_size=2, max_steps=max_steps, log_interval=1, ckpt_interval=2,
                         warmup_steps=0, gradient_accumulation_steps=2, z_loss_weight=1e-3),
        "parallelism": dict(data_parallel=1, expert_parallel=1),
        "checkpoint": dict(local_dir=str(tmp_path / "local"), remote_uri="file://" + str(tmp_path / "remote"),
                           async_workers=1, retention=3),
        "elastic": dict(min_nodes=1, max_nodes=1),
        "telemetry": dict(log_dir=str(tmp_path / "logs"), tensorboard_dir=str(tmp_path / "logs" / "tb"),
                          json_path=str(tmp_path / "logs" / "step.jsonl"), hardware_peak_tflops=1.0),
    }
    p = tmp_path / "cfg.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return p


@pytest.mark.parametrize("arch", ["toy_moe", "moe_decoder"])
def test_train_main_writes_telemetry_and_both_tiers_then_resumes(tmp_path, arch, monkeypatch):
    import train

    monkeypatch.setenv("MOE_PROFILE_DIR", str(tmp_path / "profile"))
    cfg = _write_cfg(tmp_path, arch, max_steps=4)
    assert train.main(["--config", str(cfg), "--no-wandb", "--cpu", "--profile"]) == 0
    assert len(list((tmp_path / "profile").glob("run_*_rank0.json"))) == 1
    lines = [json.loads(l) for l in (tmp_path / "logs" / "step.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines] == [0, 1, 2, 3]
    rec = lines[-1]
    for key in ("loss", "mfu", "tokens_per_sec", "kernel", "collective", "memory", "infra", "routing", "rank", "ts",
                "sparse_mfu", "dead_expert_count", "routing_efficiency", "active_experts", "dropped_token_fraction"):
        assert key in rec
    assert rec["kernel"]["used_triton"] is False and rec["infra"]["grad_accum"] == 2
    assert {"all_to_all_dispatch_ms", "all_to_all_combine_ms", "expert_compute_ms",
            "comm_compute_overlap_ratio"} <= set(rec["collective"])
    assert rec["routing"]["active_experts"] == 4 and rec["loss"] == rec["loss"]
    for tier in ("local", "remote"):
        files = sorted(str(p.relative_to(tmp_path / tier)) for p in (tmp_path / tier).rglob("*") if p.is_file())
        assert "ckpts/step=000004/rank=000000.pt" in files and "ckpts/step=000004/rank=000000.meta.json" in files
    meta = json.loads((tmp_path / "local" / "ckpts" / "step=000004" / "rank=000000.meta.json").read_text())
    assert meta["schema_version"] == 2 and meta["world_size"] == 1

    # a second run with more steps resumes after the newest checkpoint instead of starting over
    cfg = _write_cfg(tmp_path, arch, max_steps=6)
    assert train.main(["--config", str(cfg), "--no-wandb", "--cpu"]) == 0
    lines = [json.loads(l) for l in (tmp_path / "logs" / "step.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines][4:] == [5]
