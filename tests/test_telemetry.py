"""Telemetry envelope, sinks and thread safety (reference: tests/test_telemetry.py)."""

import json
import threading
import types

import pytest

import composed_mixture_of_experts_engine_b200.telemetry.logger as L
from composed_mixture_of_experts_engine_b200.telemetry.logger import (PhaseTimer, PrometheusExporter, StepRecord,
                                                                      StructuredLogger, WandBSink, overlap_ratio)

pytestmark = pytest.mark.cpu

ENVELOPE = {"step", "loss", "mfu", "tokens_per_sec", "kernel", "collective", "memory", "infra", "routing",
            "wall_clock_ms", "sparse_mfu", "dead_expert_count", "routing_efficiency", "active_experts",
            "dropped_token_fraction", "rank", "ts"}


def test_envelope_keys_and_routing_mirror(tmp_path):
    lg = StructuredLogger(str(tmp_path / "a" / "step.jsonl"), rank=3, also_stdout=False, wandb_enabled=False)
    lg.emit(StepRecord(step=1, loss=2.5, mfu=0.3, tokens_per_sec=100.0, sparse_mfu=0.01, dead_expert_count=2,
                       routing={"expert_load_imbalance": 1.2}))
    lg.close()
    lg.close()  # idempotent
    rec = json.loads((tmp_path / "a" / "step.jsonl").read_text().strip())
    assert set(rec) == ENVELOPE and rec["rank"] == 3
    assert rec["routing"]["sparse_mfu"] == 0.01 and rec["routing"]["dead_expert_count"] == 2
    assert rec["routing"]["expert_load_imbalance"] == 1.2


def test_concurrent_emit(tmp_path):
    lg = StructuredLogger(str(tmp_path / "s.jsonl"), rank=1, also_stdout=False, wandb_enabled=False)
    threads = [threading.Thread(target=lambda i=i: lg.emit(StepRecord(i, 1.0, 0.1, 1.0))) for i in range(100)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    lg.close()
    lines = (tmp_path / "s.jsonl").read_text().strip().splitlines()
    assert sorted(json.loads(l)["step"] for l in lines) == list(range(100))


def test_stdout_only_rank0(tmp_path, capsys):
    for rank in (0, 1):
        lg = StructuredLogger(str(tmp_path / f"r{rank}.jsonl"), rank=rank, also_stdout=True, wandb_enabled=False)
        lg.emit(StepRecord(7, 1.0, 0.1, 1.0))
        lg.close()
    out = capsys.readouterr().out.strip().splitlines()
    assert len(out) == 1 and json.loads(out[0])["rank"] == 0


def test_wandb_gating(monkeypatch):
    calls = []
    fake = types.SimpleNamespace(init=lambda **kw: calls.append(("init", kw)), log=lambda p, step: calls.append(("log", p, step)),
                                 finish=lambda: calls.append(("finish",)), run=None,
                                 config=types.SimpleNamespace(update=lambda c, allow_val_change: calls.append(("cfg", c))))
    monkeypatch.setattr(L, "_wandb_lib", fake)
    monkeypatch.setattr(L, "_HAS_WANDB", True)
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    assert not WandBSink(rank=0).active
    monkeypatch.setenv("WANDB_API_KEY", "k")
    assert not WandBSink(rank=1).active and not WandBSink(rank=0, enabled=False).active
    sink = WandBSink(rank=0, init_kwargs={"project": "p"})
    assert sink.active and calls[0] == ("init", {"project": "p"})
    sink.log(StepRecord(3, 1.5, 0.2, 9.0, collective={"all_to_all_dispatch_ms": 0.4, "name": "x"}))
    kind, payload, step = calls[-1]
    assert kind == "log" and step == 3 and payload["collective/all_to_all_dispatch_ms"] == 0.4
    assert "collective/name" not in payload and payload["routing/sparse_mfu"] == 0.0
    sink.log_config({"a": 1})
    sink.finish()
    assert not sink.active


def test_prometheus_disabled_off_rank0():
    exp = PrometheusExporter(port=0, rank=1)
    exp.update(StepRecord(0, 1.0, 0.1, 1.0))  # no-op, must not raise


def test_phase_timer_cpu_and_overlap():
    t = PhaseTimer()
    with t.phase("a"):
        sum(range(1000))
    with t.phase("a"):
        pass
    got = t.resolve()
    assert got["a"] > 0 and t.resolve() == {}
    off = PhaseTimer(enabled=False)
    with off.phase("x"):
        pass
    assert off.resolve() == {}
    assert overlap_ratio(1.0, 2.0, 2.0) == 1.0 and overlap_ratio(1.0, 2.0, 3.0) == 0.0
    assert overlap_ratio(0.0, 1.0, 1.0) == 0.0 and overlap_ratio(2.0, 2.0, 3.0) == 0.5


def test_pull_overlap_ratio_from_device_stamps():
    """The overlap ratio of the fused dispatch is the share of the transfer interval [first pull, last pull] that
    lies inside the tensor-core interval [first MMA, last MMA] (reference semantics of `last_overlap_ratio`:
    pkg/distributed/moe_layer.py:340-341); a launch that pulled nothing reports None."""
    import torch

    from composed_mixture_of_experts_engine_b200.ops import kernels

    i64max = kernels._I64_MAX
    t = lambda *v: torch.tensor(v, dtype=torch.int64)
    assert kernels.pull_overlap_ratio(t(100, 700, 120, 1100)) == pytest.approx(580 / 600)   # MMAs start 20 ns in
    assert kernels.pull_overlap_ratio(t(100, 700, 0, 2000)) == 1.0                          # transfer fully covered
    assert kernels.pull_overlap_ratio(t(100, 700, 800, 900)) == 0.0                         # disjoint intervals
    assert kernels.pull_overlap_ratio(t(100, 700, 400, 500)) == pytest.approx(100 / 600)    # MMAs inside the transfer
    assert kernels.pull_overlap_ratio(t(i64max, 0, i64max, 0)) is None                      # nothing recorded
    assert kernels.pull_overlap_ratio(t(100, 100, 50, 60)) is None                          # empty transfer interval


def test_device_clock_reader_reads_nvml_without_changing_anything(tmp_path, monkeypatch):
    """Clock, power and active clock-event reasons come from read-only NVML queries (tested against a fake NVML that
    fails on any call that is not a query); without NVML the reader returns an empty dict."""
    from composed_mixture_of_experts_engine_b200.telemetry.logger import DeviceClockReader

    class FakeNvml:
        NVML_CLOCK_SM = 1
        nvmlClocksEventReasonHwSlowdown = 0x8
        nvmlClocksEventReasonSwPowerCap = 0x4
        nvmlClocksEventReasonHwThermalSlowdown = 0x40
        nvmlClocksEventReasonSwThermalSlowdown = 0x20
        calls = []

        def nvmlInit(self):
            self.calls.append("init")

        def nvmlDeviceGetHandleByIndex(self, i):
            self.calls.append(("handle", i))
            return ("gpu", i)

        def nvmlDeviceGetClockInfo(self, h, kind):
            return 1462

        def nvmlDeviceGetMaxClockInfo(self, h, kind):
            return 1965

        def nvmlDeviceGetPowerUsage(self, h):
            return 992410  # milliwatts

        def nvmlDeviceGetCurrentClocksEventReasons(self, h):
            return 0x4

        def __getattr__(self, name):  # anything else (a setter, a reset) is a test failure
            raise AssertionError(f"unexpected NVML call {name}")

    fake = FakeNvml()
    got = DeviceClockReader(3, nvml=fake).read()
    assert got == {"sm_clock_mhz": 1462, "sm_clock_max_mhz": 1965, "power_w": 992.4,
                   "clock_event_reasons": ["sw_power_cap"]}
    assert ("handle", 3) in fake.calls

    class Broken:
        def nvmlInit(self):
            raise RuntimeError("no driver")

    assert DeviceClockReader(0, nvml=Broken()).read() == {}

    # the logger merges the reading into the infra block of a record that does not carry one already
    logger = StructuredLogger(json_path=str(tmp_path / "s.jsonl"), tensorboard_dir=None, rank=0, also_stdout=False,
                              wandb_enabled=False)
    logger._clocks = DeviceClockReader(0, nvml=fake)
    logger.emit(StepRecord(step=1, loss=1.0, mfu=0.5, tokens_per_sec=1e5, infra={"restart_count": 0}))
    logger.close()
    rec = json.loads((tmp_path / "s.jsonl").read_text().splitlines()[-1])
    assert rec["infra"]["sm_clock_mhz"] == 1462 and rec["infra"]["restart_count"] == 0
    assert rec["infra"]["clock_event_reasons"] == ["sw_power_cap"]
