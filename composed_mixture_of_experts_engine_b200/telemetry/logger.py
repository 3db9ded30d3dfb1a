"""Structured per-step telemetry: JSONL (every rank), stdout / TensorBoard / Prometheus / WandB (rank 0).

Envelope and sinks follow the reference's ``pkg/telemetry/logger.py:79-472``: ``StepRecord`` with the
``kernel / collective / memory / infra / routing`` blocks (the five MoE fields are mirrored into
``routing``), ``rank`` and ``ts`` added at emit time, 15 ``moe_*`` Prometheus gauges, WandB keys prefixed
by section, thread-safe ``emit``.  Added: :class:`PhaseTimer`, CUDA-event pairs per phase that are only
resolved when a record is emitted, so that timing a phase never makes the training thread wait for the GPU
(the reference synchronises on every event, ``pkg/distributed/expert_parallel.py:128``).
"""

from __future__ import annotations

import json
import logging
import os
import sys
import threading
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch

log = logging.getLogger(__name__)

try:  # optional sinks
    from torch.utils.tensorboard import SummaryWriter  # type: ignore

    _HAS_TB = True
except Exception:  # pragma: no cover - depends on the environment
    SummaryWriter = None  # type: ignore
    _HAS_TB = False

try:
    from prometheus_client import CollectorRegistry, Gauge, start_http_server  # type: ignore

    _HAS_PROM = True
except Exception:  # pragma: no cover
    _HAS_PROM = False

try:
    import wandb as _wandb_lib  # type: ignore

    _HAS_WANDB = True
except Exception:
    _wandb_lib = None  # type: ignore
    _HAS_WANDB = False

_MOE_FIELDS = ("sparse_mfu", "dead_expert_count", "routing_efficiency", "active_experts", "dropped_token_fraction")
_SECTIONS = ("kernel", "collective", "memory", "infra", "routing")


@dataclass
class StepRecord:
    """One training step as it goes on the wire."""

    step: int
    loss: float
    mfu: float
    tokens_per_sec: float
    kernel: dict = field(default_factory=dict)
    collective: dict = field(default_factory=dict)
    memory: dict = field(default_factory=dict)
    infra: dict = field(default_factory=dict)
    routing: dict = field(default_factory=dict)
    wall_clock_ms: float = 0.0
    sparse_mfu: float = 0.0
    dead_expert_count: int = 0
    routing_efficiency: float = 0.0
    active_experts: int = 0
    dropped_token_fraction: float = 0.0

    def __post_init__(self) -> None:
        for name in _MOE_FIELDS:
            self.routing.setdefault(name, getattr(self, name))


class DeviceClockReader:
    """Reads (never sets) the SM clock, power draw and active clock-event reasons of one GPU through NVML.

    On a power-capped part the sustained SM clock decides the step time (the same kernels ran 4 % apart on two
    boxes whose clocks settled at 1406 and 1462 MHz), so a throughput figure without the clock beside it cannot
    be compared across machines.  ``read()`` returns ``{}`` when NVML or the ``pynvml`` module is not there.
    """

    _REASONS = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown", "nvmlClocksThrottleReasonHwSlowdown"),
                ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown",
                 "nvmlClocksThrottleReasonHwThermalSlowdown"),
                ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown",
                 "nvmlClocksThrottleReasonSwThermalSlowdown"),
                ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap", "nvmlClocksThrottleReasonSwPowerCap"))

    def __init__(self, device_index: int = 0, nvml: Any = None):
        self._nvml, self._handle = None, None
        try:
            if nvml is None:
                import pynvml as nvml  # type: ignore
            nvml.nvmlInit()
            self._nvml, self._handle = nvml, nvml.nvmlDeviceGetHandleByIndex(device_index)
        except Exception:
            self._nvml = None

    def read(self) -> Dict[str, Any]:
        n, h = self._nvml, self._handle
        if n is None:
            return {}
        out: Dict[str, Any] = {}
        try:
            out["sm_clock_mhz"] = int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))
            out["sm_clock_max_mhz"] = int(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))
            out["power_w"] = round(n.nvmlDeviceGetPowerUsage(h) / 1000.0, 1)
            get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
            mask = int(get(h))
            active = []
            for name, new_const, old_const in self._REASONS:
                bit = getattr(n, new_const, None)
                if bit is None:
                    bit = getattr(n, old_const, 0)
                if mask & int(bit):
                    active.append(name)
            out["clock_event_reasons"] = active
        except Exception:
            pass
        return out


def _nvtx_enabled() -> bool:
    """``CMOE_NVTX=1`` wraps every timed phase (and the trainer's microbatches / optimizer step) in an NVTX range."""
    return os.environ.get("CMOE_NVTX", "0") not in ("", "0") and torch.cuda.is_available()


class PhaseTimer:
    """Named CUDA-event pairs, resolved lazily.

    ``with timer.phase("dispatch"):`` records two events on the current stream and returns at once.
    ``resolve()`` (called when a record is emitted, normally many steps later) turns every finished
    pair into milliseconds, summed per name.  On CPU the host clock is used.
    """

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self._pending: List[Tuple[str, Any, Any]] = []
        self._host: Dict[str, float] = {}

    class _Ctx:
        def __init__(self, timer: "PhaseTimer", name: str):
            self.t, self.name = timer, name

        def __enter__(self):
            self.nvtx = _nvtx_enabled()
            if self.nvtx:  # a named range in Nsight Systems / CUPTI timelines, independent of the event timing
                torch.cuda.nvtx.range_push(self.name)
            if not self.t.enabled:
                return self
            if torch.cuda.is_available():
                self.start = torch.cuda.Event(enable_timing=True)
                self.end = torch.cuda.Event(enable_timing=True)
                self.start.record()
            else:
                self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            if not self.t.enabled:
                return False
            if torch.cuda.is_available():
                self.end.record()
                self.t._pending.append((self.name, self.start, self.end))
            else:
                self.t._host[self.name] = self.t._host.get(self.name, 0.0) + (time.perf_counter() - self.t0) * 1e3
            return False

    def phase(self, name: str) -> "PhaseTimer._Ctx":
        return PhaseTimer._Ctx(self, name)

    def resolve(self, wait: bool = False) -> Dict[str, float]:
        out = dict(self._host)
        self._host = {}
        keep = []
        for name, s, e in self._pending:
            if wait:
                e.synchronize()
            if e.query():
                out[name] = out.get(name, 0.0) + s.elapsed_time(e)
            else:
                keep.append((name, s, e))
        self._pending = keep
        return out


def overlap_ratio(comm_ms: float, compute_ms: float, fused_ms: float) -> float:
    """Fraction of the communication time hidden under compute: (comm + compute - fused) / comm in [0, 1]."""
    if comm_ms <= 0.0:
        return 0.0
    return max(0.0, min(1.0, (comm_ms + compute_ms - fused_ms) / comm_ms))


class WandBSink:
    """``wandb.log`` wrapper; active only on rank 0 with the package installed and ``WANDB_API_KEY`` set."""

    def __init__(self, rank: int = 0, enabled: bool = True, init_kwargs: Optional[Dict[str, Any]] = None):
        self._active = False
        if not enabled or rank != 0 or not _HAS_WANDB or not os.environ.get("WANDB_API_KEY"):
            return
        try:
            kwargs: Dict[str, Any] = {"project": "moe-engine"}
            kwargs.update(init_kwargs or {})
            _wandb_lib.init(**kwargs)
            self._active = True
        except Exception as exc:  # pragma: no cover - network dependent
            log.warning("WandB init failed (%s); sink disabled", exc)

    @property
    def active(self) -> bool:
        return self._active

    def log(self, record: StepRecord) -> None:
        if not self._active:
            return
        payload: Dict[str, Any] = {
            "loss": record.loss,
            "mfu": record.mfu,
            "tokens_per_sec": record.tokens_per_sec,
            "wall_clock_ms": record.wall_clock_ms,
        }
        for section in _SECTIONS:
            for k, v in getattr(record, section).items():
                if isinstance(v, (int, float)):
                    payload[f"{section}/{k}"] = v
        try:
            _wandb_lib.log(payload, step=record.step)
        except Exception as exc:
            log.warning("wandb.log failed at step %d: %s", record.step, exc)

    def log_config(self, cfg: Dict[str, Any]) -> None:
        if not self._active:
            return
        try:
            _wandb_lib.config.update(cfg, allow_val_change=True)
        except Exception as exc:
            log.warning("wandb.config.update failed: %s", exc)

    def finish(self) -> None:
        if not self._active:
            return
        try:
            _wandb_lib.finish()
        except Exception:
            pass
        self._active = False


_GAUGES = [
    ("moe_step_loss", "Training loss per step"),
    ("moe_mfu", "Model FLOPs utilisation"),
    ("moe_tokens_per_sec", "Training throughput (tokens/s)"),
    ("moe_all_to_all_dispatch_ms", "Expert-parallel dispatch latency (ms)"),
    ("moe_all_to_all_combine_ms", "Expert-parallel combine latency (ms)"),
    ("moe_expert_compute_ms", "Expert FFN compute latency (ms)"),
    ("moe_comm_compute_overlap_ratio", "Share of communication hidden under compute"),
    ("moe_peak_memory_gb", "Peak CUDA memory allocated (GB)"),
    ("moe_sparse_mfu", "MFU scaled by K/E"),
    ("moe_dead_expert_count", "Experts that received no token this step"),
    ("moe_routing_efficiency", "Fraction of the expert capacity in use"),
    ("moe_active_experts", "Experts that received at least one token"),
    ("moe_dropped_token_fraction", "Fraction of (token, slot) pairs dropped by capacity"),
    ("moe_expert_load_imbalance", "Router load imbalance (max / mean)"),
    ("moe_router_z_loss", "Router z-loss"),
]


class PrometheusExporter:
    """In-process ``/metrics`` endpoint (rank 0 only) with the fifteen ``moe_*`` gauges."""

    def __init__(self, port: int = 9102, rank: int = 0):
        self._enabled = bool(_HAS_PROM and rank == 0)
        if not self._enabled:
            return
        self._reg = CollectorRegistry()
        self._g = {name: Gauge(name, doc, registry=self._reg) for name, doc in _GAUGES}
        try:
            start_http_server(port, registry=self._reg)
        except Exception as exc:
            log.warning("could not start the Prometheus endpoint on :%d (%s)", port, exc)
            self._enabled = False

    def update(self, rec: StepRecord) -> None:
        if not self._enabled:
            return
        g = self._g
        g["moe_step_loss"].set(rec.loss)
        g["moe_mfu"].set(rec.mfu)
        g["moe_tokens_per_sec"].set(rec.tokens_per_sec)
        c = rec.collective
        g["moe_all_to_all_dispatch_ms"].set(c.get("all_to_all_dispatch_ms", 0.0))
        g["moe_all_to_all_combine_ms"].set(c.get("all_to_all_combine_ms", 0.0))
        g["moe_expert_compute_ms"].set(c.get("expert_compute_ms", 0.0))
        g["moe_comm_compute_overlap_ratio"].set(c.get("comm_compute_overlap_ratio", 0.0))
        if rec.memory:
            g["moe_peak_memory_gb"].set(rec.memory.get("peak_allocated_gb", 0.0))
        r = rec.routing or {}
        for name in _MOE_FIELDS:
            if name in r:
                g[f"moe_{name}"].set(r[name])
        if r:
            g["moe_expert_load_imbalance"].set(r.get("expert_load_imbalance", 1.0))
            g["moe_router_z_loss"].set(r.get("router_z_loss", 0.0))


class StructuredLogger:
    """Fans one :class:`StepRecord` out to every configured sink."""

    def __init__(
        self,
        json_path: str,
        tensorboard_dir: Optional[str] = None,
        rank: int = 0,
        also_stdout: bool = True,
        prometheus_port: int = 0,
        wandb_enabled: bool = True,
        wandb_init_kwargs: Optional[Dict[str, Any]] = None,
    ):
        self.rank = rank
        self.also_stdout = also_stdout
        self.json_path = Path(json_path)
        self.json_path.parent.mkdir(parents=True, exist_ok=True)
        self._fh = self.json_path.open("a", buffering=1)
        self._lock = threading.RLock()
        self._closed = False
        self._tb = None
        if _HAS_TB and tensorboard_dir and rank == 0:
            Path(tensorboard_dir).mkdir(parents=True, exist_ok=True)
            self._tb = SummaryWriter(log_dir=tensorboard_dir)
        self._peak_mem_prev = 0.0
        self._clocks = DeviceClockReader(torch.cuda.current_device()) if torch.cuda.is_available() else None
        self._prom = PrometheusExporter(port=prometheus_port, rank=rank) if prometheus_port > 0 else None
        self._wandb = WandBSink(rank=rank, enabled=wandb_enabled, init_kwargs=wandb_init_kwargs)

    def emit(self, record: StepRecord) -> None:
        if not record.memory and torch.cuda.is_available():
            stats = torch.cuda.memory_stats()
            alloc_gb = stats.get("allocated_bytes.all.peak", 0) / (1024**3)
            record.memory = {
                "peak_allocated_gb": round(alloc_gb, 4),
                "reserved_gb": round(stats.get("reserved_bytes.all.current", 0) / (1024**3), 4),
                "leak_delta_gb": round(alloc_gb - self._peak_mem_prev, 4),
            }
            self._peak_mem_prev = alloc_gb
        if self._clocks is not None and "sm_clock_mhz" not in record.infra:
            record.infra.update(self._clocks.read())  # clock, power, active clock-event reasons at emit time
        payload = asdict(record)
        payload["rank"] = self.rank
        payload["ts"] = time.time()
        line = json.dumps(payload, separators=(",", ":"))
        with self._lock:
            if not self._closed:
                self._fh.write(line + "\n")
            if self.also_stdout and self.rank == 0:
                sys.stdout.write(line + "\n")
                sys.stdout.flush()
            if self._tb is not None:
                self._tb.add_scalar("loss", record.loss, record.step)
                self._tb.add_scalar("mfu", record.mfu, record.step)
                self._tb.add_scalar("tokens_per_sec", record.tokens_per_sec, record.step)
                for section in _SECTIONS:
                    for k, v in getattr(record, section).items():
                        if isinstance(v, (int, float)):
                            self._tb.add_scalar(f"{section}/{k}", v, record.step)
        self._wandb.log(record)
        if self._prom is not None:
            self._prom.update(record)

    def log_config(self, cfg: Dict[str, Any]) -> None:
        self._wandb.log_config(cfg)

    def close(self) -> None:
        with self._lock:
            if not self._closed:
                try:
                    self._fh.close()
                except Exception:
                    pass
                if self._tb is not None:
                    try:
                        self._tb.close()
                    except Exception:
                        pass
                self._closed = True
        self._wandb.finish()
