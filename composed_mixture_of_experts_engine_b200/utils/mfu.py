"""Model-FLOPs-utilisation accounting for sparse (MoE) transformers.

Keeps the reference's API and formulas (``pkg/utils/mfu.py:46-288``): ``compute_mfu`` /
``compute_mfu_detailed`` (dense + K/E-weighted expert parameters, x2 or x3 with recompute, clamped to
[0, 1]), ``compute_moe_flops`` (per-token estimate, x3 for forward+backward) and the streaming
``MFUAccountant``.  Added here: ``exact_train_flops_per_token`` – a per-config FLOP model with GQA and
causal attention, used for the MFU that ``bench.py`` and ``train.py`` report against the measured peak –
and an accountant that can be fed device-measured step times instead of host wall-clock.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from typing import List, Optional

log = logging.getLogger(__name__)


@dataclass
class MFUResult:
    achieved_tflops: float
    peak_tflops: float
    mfu: float
    step_ms: float
    tokens_per_sec: float
    flops_dense: float
    flops_sparse: float


def _mfu_parts(batch_tokens, param_dense, param_expert, num_experts, top_k, activation_recompute):
    mult = 3.0 if activation_recompute else 2.0
    dense = mult * batch_tokens * param_dense
    sparse = mult * batch_tokens * (top_k / max(num_experts, 1)) * param_expert
    return dense, sparse


def compute_mfu_detailed(
    batch_tokens: int,
    param_dense: int,
    param_expert: int,
    num_experts: int,
    top_k: int,
    world_size: int,
    hardware_peak_tflops: float,
    step_time_sec: float,
    activation_recompute: bool = False,
) -> MFUResult:
    dense, sparse = _mfu_parts(batch_tokens, param_dense, param_expert, num_experts, top_k, activation_recompute)
    achieved = (dense + sparse) / step_time_sec / 1e12
    peak_total = world_size * hardware_peak_tflops
    mfu = max(0.0, min(1.0, achieved / max(peak_total, 1e-9)))
    return MFUResult(
        achieved_tflops=achieved,
        peak_tflops=peak_total,
        mfu=mfu,
        step_ms=step_time_sec * 1000.0,
        tokens_per_sec=batch_tokens / max(step_time_sec, 1e-9),
        flops_dense=dense,
        flops_sparse=sparse,
    )


def compute_mfu(
    batch_tokens: int,
    param_dense: int,
    param_expert: int,
    num_experts: int,
    top_k: int,
    world_size: int,
    hardware_peak_tflops: float,
    step_time_sec: float,
    activation_recompute: bool = False,
) -> float:
    res = compute_mfu_detailed(
        batch_tokens, param_dense, param_expert, num_experts, top_k, world_size, hardware_peak_tflops,
        step_time_sec, activation_recompute,
    )
    if res.mfu < 0.25:
        log.debug("MFU=%.2f%% is low (world=%d, step_ms=%.1f, tokens=%d)", res.mfu * 100, world_size, res.step_ms,
                  batch_tokens)
    elif res.mfu > 0.87:
        log.debug("MFU=%.2f%% is suspiciously high; check hardware_peak_tflops=%.0f", res.mfu * 100,
                  hardware_peak_tflops)
    return res.mfu


def compute_moe_flops(
    hidden_dim: int,
    num_layers: int,
    ffn_dim: int,
    num_experts: int,
    top_k: int,
    seq_length: int,
    batch_tokens: int,
    vocab_size: int = 0,
) -> int:
    """The reference's estimate: 3 x forward, with 4H^2 + 4HS attention, HE router, 6HFK experts, 2HV head."""
    H, F, E, K, S = hidden_dim, ffn_dim, num_experts, top_k, seq_length
    per_layer = (4 * H * H + 4 * H * S) + H * E + K * 6 * H * F
    fwd = num_layers * per_layer + (2 * H * vocab_size if vocab_size else 0)
    return 3 * fwd * batch_tokens


def exact_train_flops_per_token(
    hidden_dim: int,
    num_layers: int,
    ffn_dim: int,
    num_experts: int,
    top_k: int,
    seq_length: int,
    vocab_size: int,
    num_heads: int = 0,
    num_kv_heads: int = 0,
    head_dim: int = 0,
    attention: bool = True,
    causal: bool = True,
) -> float:
    """Forward+backward matmul FLOPs per token (backward = 2 x forward), GQA and causal masking included."""
    H, F, E, K, S = hidden_dim, ffn_dim, num_experts, top_k, seq_length
    per_layer = 2 * H * E + K * 3 * 2 * H * F  # router + gate/up/down of K experts
    if attention:
        nh = num_heads or max(1, H // 128)
        nkv = num_kv_heads or nh
        hd = head_dim or H // nh
        qkv_out = 2 * H * (nh * hd + 2 * nkv * hd) + 2 * nh * hd * H
        scores = 2 * 2 * nh * hd * S * (0.5 if causal else 1.0)  # QK^T and PV against S (or S/2) keys
        per_layer += qkv_out + scores
    fwd = num_layers * per_layer + 2 * H * vocab_size
    return 3.0 * fwd


class MFUAccountant:
    """Streaming MFU tracker: ``start_step()`` / ``end_step(tokens[, step_time_sec])`` once per step.

    ``peak_tflops`` is the peak of everything that contributed the tokens (per rank when the tokens
    are per rank, as in the reference's train loop; whole job when ``world_size`` is folded in by the
    caller).  Passing ``step_time_sec`` (e.g. from CUDA events) overrides the host timer.
    """

    def __init__(self, peak_tflops: float, mfu_target: float = 0.55, smoothing_window: int = 50):
        self.peak_tflops = peak_tflops
        self.mfu_target = mfu_target
        self.smoothing_window = smoothing_window
        self._t0 = 0.0
        self._flops_per_token: float = 0
        self.history: List[MFUResult] = []
        self._running_mfu = 0.0
        self._steps = 0
        self._window: List[float] = []

    def configure(self, flops_per_token: float) -> None:
        self._flops_per_token = flops_per_token

    def start_step(self) -> None:
        self._t0 = time.perf_counter()

    def end_step(self, tokens: int, step_time_sec: Optional[float] = None) -> MFUResult:
        dt = step_time_sec if step_time_sec is not None else (time.perf_counter() - self._t0)
        dt = max(dt, 1e-9)
        achieved = self._flops_per_token * tokens / dt / 1e12
        mfu = max(0.0, min(1.0, achieved / max(self.peak_tflops, 1e-9)))
        res = MFUResult(achieved, self.peak_tflops, mfu, dt * 1000.0, tokens / dt, 0.0, 0.0)
        self.history.append(res)
        self._steps += 1
        self._running_mfu += (mfu - self._running_mfu) / self._steps
        self._window.append(mfu)
        if len(self._window) > self.smoothing_window:
            self._window.pop(0)
        return res

    @property
    def running_mfu(self) -> float:
        return self._running_mfu

    @property
    def smoothed_mfu(self) -> float:
        return sum(self._window) / len(self._window) if self._window else 0.0

    def is_above_target(self) -> bool:
        return self._running_mfu >= self.mfu_target

    def summary_str(self) -> str:
        if not self.history:
            return "MFU: no data"
        last = self.history[-1]
        return (
            f"MFU={self._running_mfu:.2%} (smooth={self.smoothed_mfu:.2%}) | {last.tokens_per_sec:,.0f} tok/s "
            f"| step={last.step_ms:.1f}ms | {last.achieved_tflops:.2f}/{self.peak_tflops:.0f} TFLOPs"
        )
