"""MFU formulas and the streaming accountant (reference: tests/test_mfu.py, tests/test_mfu_v02.py)."""

import pytest

from composed_mixture_of_experts_engine_b200.utils.mfu import (MFUAccountant, compute_mfu, compute_mfu_detailed,
                                                               compute_moe_flops, exact_train_flops_per_token)

pytestmark = pytest.mark.cpu
KW = dict(batch_tokens=4096, param_dense=10**8, param_expert=10**9, num_experts=64, top_k=2, world_size=8,
          hardware_peak_tflops=989.0, step_time_sec=1.0)


def test_scaling_laws():
    base = compute_mfu(**KW)
    assert 0 < base < 1
    assert compute_mfu(**{**KW, "batch_tokens": 8192}) == pytest.approx(2 * base)
    assert compute_mfu(**{**KW, "world_size": 16}) == pytest.approx(base / 2)
    assert compute_mfu(**{**KW, "step_time_sec": 2.0}) == pytest.approx(base / 2)
    assert compute_mfu(**{**KW, "activation_recompute": True}) == pytest.approx(1.5 * base)


def test_clamped_and_detailed():
    assert compute_mfu(**{**KW, "step_time_sec": 1e-9}) == 1.0
    d = compute_mfu_detailed(**KW)
    assert d.flops_dense == 2.0 * 4096 * 10**8
    assert d.flops_sparse == pytest.approx(2.0 * 4096 * (2 / 64) * 10**9)
    assert d.tokens_per_sec == pytest.approx(4096) and d.peak_tflops == 8 * 989.0


def test_reference_flop_estimate():
    got = compute_moe_flops(hidden_dim=64, num_layers=2, ffn_dim=128, num_experts=4, top_k=2, seq_length=16,
                            batch_tokens=10, vocab_size=256)
    per_layer = 4 * 64 * 64 + 4 * 64 * 16 + 64 * 4 + 2 * 6 * 64 * 128
    assert got == 3 * (2 * per_layer + 2 * 64 * 256) * 10


def test_exact_flops_olmoe_order_of_magnitude():
    f = exact_train_flops_per_token(2048, 16, 1024, 64, 8, 4096, 50304, 16, 16, 128)
    assert 7.0e9 < f < 9.0e9  # ~6 x 1.18 B active parameters + causal attention


def test_accountant_history_and_window():
    acc = MFUAccountant(peak_tflops=1000.0, mfu_target=0.5, smoothing_window=3)
    acc.configure(flops_per_token=10**9)
    for i in range(5):
        acc.start_step()
        r = acc.end_step(tokens=1000 * (i + 1), step_time_sec=0.01)
    assert len(acc.history) == 5 and len(acc._window) == 3
    assert r.mfu == pytest.approx(10**9 * 5000 / 0.01 / 1e12 / 1000.0)
    assert acc.smoothed_mfu == pytest.approx(sum(h.mfu for h in acc.history[-3:]) / 3)
    assert acc.running_mfu == pytest.approx(sum(h.mfu for h in acc.history) / 5)
    assert "tok/s" in acc.summary_str() and not acc.is_above_target()
    assert MFUAccountant(1.0).summary_str() == "MFU: no data"


def test_memory_plan_matches_the_model_arithmetic_and_a_measured_peak():
    """Parameter totals of the two full-size configurations (6.92 B and 46.7 B) and the one-GPU plan of the
    OLMoE-shaped model against the peak allocation measured on a B200 (154.7 GB at micro-batch 4)."""
    from pathlib import Path

    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig
    from composed_mixture_of_experts_engine_b200.utils.memory import format_plan, parameter_counts, plan_memory

    configs = Path(__file__).resolve().parent.parent / "configs"
    olmoe = MoEConfig.from_yaml(configs / "olmoe_1b7b.yaml")
    mixtral = MoEConfig.from_yaml(configs / "mixtral_8x7b.yaml")
    assert parameter_counts(olmoe)["total"] / 1e9 == pytest.approx(6.92, abs=0.01)
    assert parameter_counts(olmoe)["active_per_token"] / 1e9 == pytest.approx(1.18, abs=0.01)
    assert parameter_counts(mixtral)["total"] / 1e9 == pytest.approx(46.7, abs=0.05)
    d = olmoe.to_dict()
    d["parallelism"].update(data_parallel=1, expert_parallel=1)
    one = plan_memory(MoEConfig.from_dict(d), 1)
    assert one["total_gb"] == pytest.approx(154.7, rel=0.05) and one["fits"]
    eight = plan_memory(olmoe, 8)
    assert eight["total_gb"] < one["total_gb"] / 2 and eight["ep_buffers_gb"] > 0
    plan = plan_memory(mixtral, 8)
    assert plan["fits"] and plan["params_local_b"] == pytest.approx(46.7 / 8, rel=0.05)
    assert "fits" in format_plan(plan)
    d = mixtral.to_dict()
    d["parallelism"].update(data_parallel=1, expert_parallel=1, tensor_parallel=1, pipeline_parallel=1)
    assert not plan_memory(MoEConfig.from_dict(d), 1)["fits"]
