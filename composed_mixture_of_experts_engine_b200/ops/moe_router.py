"""Top-k softmax router: module, autograd function, functional entry point and the fp64 oracle.

Public surface of the reference's ``pkg/kernels/moe_router.py`` (``MoERouter``, ``MoERouterFunction`` /
``MoERouterAutograd``, ``moe_topk_route``, ``RouterProfile``, ``_reference_route_fp64``,
``_reference_backward_fp64``, ``_compute_load_imbalance``, ``_compute_router_z_loss``,
``_should_use_triton``, ``MIN_TRITON_DIM``, ``TRITON_AVAILABLE``).

On a CUDA device with bf16 tokens the whole forward is ONE sm_100a kernel (gate GEMM on tcgen05,
softmax, top-k, renormalisation, per-expert counts, load-balance sums, z-loss); the backward is one
elementwise kernel plus two tcgen05 GEMMs.  There is no Triton path (``TRITON_AVAILABLE`` is False and
``RouterProfile.used_triton`` is always False; ``used_fused_kernel`` says whether the sm_100a kernel ran).
Everywhere else (CPU, fp32 tokens, shapes the kernel does not cover) the fp64 PyTorch restatement runs;
it is also the test oracle.

Unlike the reference (``moe_router.py:690-734``) the module makes no host round trip per call: counts,
z-loss and the conservation check are produced on the device and only read when ``last_profile`` is.
The load-balance loss ``E * sum_i f_i * P_i`` and the z-loss are returned as differentiable tensors
(``last_aux_loss`` / ``last_z_loss``); the reference only had a non-differentiable z-loss float.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import _ext

TRITON_AVAILABLE = False  # there is no Triton path in this package
MIN_TRITON_DIM = 16       # smallest N/H/E for which the reference dispatched its device kernel
MAX_FUSED_EXPERTS = 256
MAX_FUSED_TOPK = 8

__all__ = [
    "MoERouter",
    "MoERouterFunction",
    "MoERouterAutograd",
    "moe_topk_route",
    "RouterProfile",
    "TRITON_AVAILABLE",
]


# --------------------------------------------------------------------------------------------------
# fp64 oracle (also the CPU production path)
# --------------------------------------------------------------------------------------------------
def _reference_route_fp64(tokens: torch.Tensor, gate_w: torch.Tensor, k: int
                          ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(topk_idx int64 [N,K], topk_w [N,K], logits [N,E]) computed in float64, cast back to the token dtype."""
    logits = tokens.to(torch.float64) @ gate_w.to(torch.float64)
    probs = torch.softmax(logits, dim=-1)
    vals, idx = torch.topk(probs, k=k, dim=-1, largest=True)
    w = vals / vals.sum(dim=-1, keepdim=True).clamp_min(1e-30)
    return idx.to(torch.long), w.to(tokens.dtype), logits.to(tokens.dtype)


def _reference_backward_fp64(logits: torch.Tensor, topk_idx: torch.Tensor, grad_w: torch.Tensor, k: int, E: int
                             ) -> torch.Tensor:
    """d(sum grad_w * w)/d(logits) in float64: through the renormalisation, the gather and the softmax."""
    probs = torch.softmax(logits.to(torch.float64), dim=-1)
    v = probs.gather(1, topk_idx)
    S = v.sum(dim=-1, keepdim=True).clamp_min(1e-30)
    gw = grad_w.to(torch.float64)
    grad_v = gw / S - (gw * v).sum(dim=-1, keepdim=True) / (S * S)
    grad_p = torch.zeros_like(probs).scatter_add_(1, topk_idx, grad_v)
    return probs * (grad_p - (grad_p * probs).sum(dim=-1, keepdim=True))


def _compute_load_imbalance(dispatch_cnt: torch.Tensor) -> float:
    cnt = dispatch_cnt.float()
    mean = float(cnt.mean())
    return 1.0 if mean < 1e-9 else float(cnt.max()) / mean


def _compute_router_z_loss(logits: torch.Tensor) -> float:
    return float((torch.logsumexp(logits.float(), dim=-1) ** 2).mean())


def _should_use_fused(tokens: torch.Tensor, gate_w: torch.Tensor, force_reference: bool, k: int = 1) -> bool:
    """Single source of truth for "will the sm_100a kernel run" (used for dispatch and for telemetry)."""
    if force_reference or not (tokens.is_cuda and gate_w.is_cuda):
        return False
    import os

    if os.environ.get("CMOE_FORCE_LIBRARY", "0") == "1":  # the benchmarks' library arm: no device code of this package
        return False
    if tokens.dtype != torch.bfloat16 or tokens.dim() != 2:
        return False
    N, H = tokens.shape
    E = gate_w.shape[1]
    return (N >= 1 and H % 8 == 0 and E % 8 == 0 and E <= MAX_FUSED_EXPERTS and 1 <= k <= min(MAX_FUSED_TOPK, E)
            and tokens.stride(1) == 1 and (tokens.stride(0) * 2) % 16 == 0)


def _next_pow2(n: int) -> int:
    """Smallest power of two >= n (the reference sizes its expert tile with it, moe_router.py:297-388; the fused
    kernel pads the expert dimension to a multiple of 16 instead, this stays for callers of the helper)."""
    return 1 if n <= 1 else 1 << (int(n) - 1).bit_length()


def _should_use_triton(tokens: torch.Tensor, gate_w: torch.Tensor, force_reference: bool) -> bool:
    """Kept for callers of the reference API: true when a device kernel (here: the fused sm_100a one) runs."""
    return _should_use_fused(tokens, gate_w, force_reference)


# --------------------------------------------------------------------------------------------------
# fused device path
# --------------------------------------------------------------------------------------------------
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _router_workspace(device: torch.device, E: int) -> torch.Tensor:
    key = (device.index or 0, E)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(3 * E + 4, dtype=torch.int32, device=device)  # csrc/router.cuh: router_workspace_words
        _workspaces[key] = ws
    return ws


class RouterOutput:
    """Everything the fused forward produced, all on the device."""

    __slots__ = ("idx32", "w32", "logits", "lse", "counts", "mean_prob", "stats", "events")

    def __init__(self, idx32, w32, logits, lse, counts, mean_prob, stats, events=None):
        self.idx32, self.w32, self.logits, self.lse = idx32, w32, logits, lse
        self.counts, self.mean_prob, self.stats, self.events = counts, mean_prob, stats, events


def fused_router_forward(tokens: torch.Tensor, gate_w_bf16: torch.Tensor, k: int, timed: bool = False) -> RouterOutput:
    from .kernels import status_word

    N, _ = tokens.shape
    E = gate_w_bf16.shape[1]
    dev = tokens.device
    f32 = dict(device=dev, dtype=torch.float32)
    out = RouterOutput(
        torch.empty(N, k, device=dev, dtype=torch.int32), torch.empty(N, k, **f32), torch.empty(N, E, **f32),
        torch.empty(N, **f32), torch.empty(E, device=dev, dtype=torch.int32), torch.empty(E, **f32),
        torch.empty(4, **f32),
    )
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    _ext.ext().router_fwd(tokens, gate_w_bf16, k, out.logits, out.idx32, out.w32, out.lse, out.counts, out.mean_prob,
                          out.stats, _router_workspace(dev, E), status_word(dev), 0)
    if timed:
        e1.record()
        out.events = (e0, e1)
    return out


class FusedRouterFunction(torch.autograd.Function):
    """(tokens, gate_w) -> (gate weights fp32 [N,K], aux loss, z loss); indices and statistics ride on ``holder``."""

    @staticmethod
    def forward(ctx, tokens, gate_w, k: int, holder: Dict[str, Any], timed: bool):
        gw16 = gate_w if gate_w.dtype == torch.bfloat16 else gate_w.to(torch.bfloat16)
        gw16 = gw16.contiguous()
        out = fused_router_forward(tokens, gw16, k, timed)
        holder["out"] = out
        ctx.save_for_backward(tokens, gw16, out.logits, out.lse, out.idx32, out.counts)
        ctx.gate_dtype = gate_w.dtype
        ctx.mark_non_differentiable(out.idx32)
        return out.w32, out.stats[0], out.stats[1], out.idx32

    @staticmethod
    def backward(ctx, grad_w, grad_aux, grad_z, _grad_idx):
        from .kernels import linear_nt, linear_tn

        tokens, gw16, logits, lse, idx32, counts = ctx.saved_tensors
        N, E = logits.shape
        gl16 = torch.empty(N, E, device=logits.device, dtype=torch.bfloat16)
        gw = None if grad_w is None else grad_w.float().contiguous()
        ga = None if grad_aux is None else grad_aux.float().reshape(1).contiguous()
        gz = None if grad_z is None else grad_z.float().reshape(1).contiguous()
        _ext.ext().router_bwd(logits, lse, idx32, gw, counts, ga, gz, gl16, None)
        grad_tokens = grad_gate = None
        if ctx.needs_input_grad[0]:
            grad_tokens = linear_nt(gl16, gw16)  # [N, E] x [H, E]^T
        if ctx.needs_input_grad[1]:
            grad_gate = linear_tn(tokens, gl16).to(ctx.gate_dtype)  # tokens^T [H, N] x gl [N, E]
        return grad_tokens, grad_gate, None, None, None


# --------------------------------------------------------------------------------------------------
# autograd function with the reference's signature
# --------------------------------------------------------------------------------------------------
class MoERouterFunction(torch.autograd.Function):
    """``apply(tokens[N,H], gate_w[H,E], k, force_reference=False, report=None) -> (idx int64, w)``."""

    @staticmethod
    def forward(ctx, tokens, gate_w, k: int, force_reference: bool = False, report: Optional[dict] = None):
        N, H = tokens.shape
        E = gate_w.shape[1]
        fused = _should_use_fused(tokens, gate_w, force_reference, k)
        if fused:
            gw16 = gate_w.to(torch.bfloat16).contiguous()
            out = fused_router_forward(tokens, gw16, k, timed=report is not None)
            idx, w, logits = out.idx32.long(), out.w32.to(tokens.dtype), out.logits
            ctx.fused_saved = (gw16, out.lse, out.idx32, out.counts)
            if report is not None:
                report["output"] = out
        else:
            idx, w, logits = _reference_route_fp64(tokens, gate_w, k)
            ctx.fused_saved = None
        if report is not None:
            report["used_fused_kernel"] = fused
            report["used_triton"] = False
            report["logits"] = logits
        ctx.save_for_backward(tokens, gate_w, logits, idx)
        ctx.k, ctx.E, ctx.fused = k, E, fused
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _grad_idx, grad_w):
        tokens, gate_w, logits, idx = ctx.saved_tensors
        if ctx.fused:
            from .kernels import linear_nt, linear_tn

            gw16, lse, idx32, counts = ctx.fused_saved
            gl16 = torch.empty(logits.shape, device=logits.device, dtype=torch.bfloat16)
            _ext.ext().router_bwd(logits, lse, idx32, grad_w.float().contiguous(), counts, None, None, gl16, None)
            grad_tokens = linear_nt(gl16, gw16).to(tokens.dtype) if ctx.needs_input_grad[0] else None
            grad_gate = linear_tn(tokens, gl16).to(gate_w.dtype) if ctx.needs_input_grad[1] else None
            return grad_tokens, grad_gate, None, None, None
        gl = _reference_backward_fp64(logits, idx, grad_w, ctx.k, ctx.E)
        grad_tokens = (gl @ gate_w.to(torch.float64).t()).to(tokens.dtype) if ctx.needs_input_grad[0] else None
        grad_gate = (tokens.to(torch.float64).t() @ gl).to(gate_w.dtype) if ctx.needs_input_grad[1] else None
        return grad_tokens, grad_gate, None, None, None


MoERouterAutograd = MoERouterFunction


def moe_topk_route(tokens: torch.Tensor, gate_w: torch.Tensor, k: int, force_reference: bool = False
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Route ``[B,S,H]`` or ``[N,H]`` tokens; returns ``(idx int64 [N,K], w [N,K])``."""
    if tokens.dim() == 3:
        tokens = tokens.reshape(-1, tokens.shape[-1])
    elif tokens.dim() != 2:
        raise ValueError(f"tokens must be [B,S,H] or [N,H], got shape {list(tokens.shape)}")
    if not (1 <= k <= gate_w.shape[1]):
        raise ValueError(f"k={k} must be in [1, {gate_w.shape[1]}]")
    return MoERouterFunction.apply(tokens, gate_w, k, force_reference, None)


# --------------------------------------------------------------------------------------------------
# module
# --------------------------------------------------------------------------------------------------
def _fused_stage_bytes(num_experts: int) -> int:
    """Shared memory of one pipeline stage of the fused router kernel (csrc/router.cu): a 128-token x 64-wide bf16
    slice of the activations plus the matching slice of the gate weights, experts padded to a multiple of 64.
    Reported on every path as the on-chip working set per block, like the reference's theoretical figure
    (pkg/kernels/moe_router.py:703-714)."""
    e_chunks = max(1, (num_experts + 63) // 64)
    return 128 * 64 * 2 + e_chunks * 64 * 64 * 2


@dataclass
class RouterProfile:
    sram_bytes_per_block: int = 0
    achieved_bandwidth_gbps: float = 0.0
    kernel_ms: float = 0.0
    used_triton: bool = False
    tokens_per_expert_mean: float = 0.0
    tokens_per_expert_std: float = 0.0
    expert_load_imbalance: float = 1.0
    router_z_loss: float = 0.0
    used_fused_kernel: bool = False
    backend: str = "torch-fp64"
    aux_loss: float = 0.0
    dispatch_counts: Optional[list] = None


class MoERouter(nn.Module):
    """Learned top-k router.  ``forward(tokens[N,H]) -> (idx int64 [N,K], w [N,K], dispatch_cnt int64 [E])``."""

    def __init__(self, hidden_dim: int, num_experts: int, top_k: int = 2, bias: bool = False,
                 dtype: torch.dtype = torch.float32):
        super().__init__()
        if not (1 <= top_k <= num_experts):
            raise ValueError(f"top_k={top_k} must be in [1, num_experts={num_experts}]")
        self.hidden_dim, self.num_experts, self.top_k = hidden_dim, num_experts, top_k
        self.gate_w = nn.Parameter(torch.empty(hidden_dim, num_experts, dtype=dtype))
        nn.init.normal_(self.gate_w, mean=0.0, std=1.0 / math.sqrt(hidden_dim))
        self.bias = nn.Parameter(torch.zeros(num_experts, dtype=dtype)) if bias else None
        self.profile_timing = False  # record CUDA events around the kernel (resolved lazily)
        self._pending: Optional[dict] = None
        self._profile: Optional[RouterProfile] = None
        self._last_logits: Optional[torch.Tensor] = None
        self.last_aux_loss: Optional[torch.Tensor] = None
        self.last_z_loss: Optional[torch.Tensor] = None
        self.last_idx32: Optional[torch.Tensor] = None
        self.last_w32: Optional[torch.Tensor] = None

    def extra_repr(self) -> str:
        return f"hidden_dim={self.hidden_dim}, num_experts={self.num_experts}, top_k={self.top_k}"

    # the statistics of the last call are materialised (one device read) only when somebody asks
    @property
    def last_profile(self) -> Optional[RouterProfile]:
        if self._pending is not None:
            self._profile = self._materialise(self._pending)
            self._pending = None
        return self._profile

    @last_profile.setter
    def last_profile(self, value: Optional[RouterProfile]) -> None:
        self._pending, self._profile = None, value

    def _materialise(self, pend: dict) -> RouterProfile:
        counts = pend["counts"].detach().to("cpu", torch.float64)
        N, H, E, K = pend["N"], self.hidden_dim, self.num_experts, self.top_k
        total = int(counts.sum())
        if total != N * K:
            raise RuntimeError(
                f"Token conservation violation: dispatched {total} (token, slot) pairs, expected {N * K} "
                f"(N={N}, K={K})")
        kernel_ms = 0.0
        if pend.get("events") is not None:
            e0, e1 = pend["events"]
            e1.synchronize()
            kernel_ms = e0.elapsed_time(e1)
        bytes_moved = N * H * pend["elem"] + H * E * pend["elem"] + N * E * 4 + N * K * 8
        z = float(pend["z_loss"]) if pend.get("z_loss") is not None else 0.0
        aux = float(pend["aux_loss"]) if pend.get("aux_loss") is not None else 0.0
        mean = float(counts.mean())
        return RouterProfile(
            sram_bytes_per_block=_fused_stage_bytes(E),
            achieved_bandwidth_gbps=(bytes_moved / (kernel_ms * 1e6)) if kernel_ms > 0 else 0.0,
            kernel_ms=kernel_ms,
            used_triton=False,
            tokens_per_expert_mean=mean,
            tokens_per_expert_std=float(counts.std(unbiased=False)) if E > 1 else 0.0,
            expert_load_imbalance=(float(counts.max()) / mean) if mean > 1e-9 else 1.0,
            router_z_loss=z,
            used_fused_kernel=pend["fused"],
            backend="sm100a-fused" if pend["fused"] else "torch-fp64",
            aux_loss=aux,
            dispatch_counts=[int(c) for c in counts.tolist()],
        )

    def forward(self, tokens: torch.Tensor, force_reference: bool = False
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if tokens.dim() == 3:
            tokens = tokens.reshape(-1, tokens.shape[-1])
        if tokens.dim() != 2 or tokens.shape[1] != self.hidden_dim:
            raise ValueError(f"expected tokens [N, {self.hidden_dim}], got {list(tokens.shape)}")
        N = tokens.shape[0]
        E, K = self.num_experts, self.top_k
        fused = self.bias is None and _should_use_fused(tokens, self.gate_w, force_reference, K)
        if fused:
            holder: Dict[str, Any] = {}
            w32, aux, z, idx32 = FusedRouterFunction.apply(tokens, self.gate_w, K, holder, self.profile_timing)
            out: RouterOutput = holder["out"]
            idx, w, counts = idx32.long(), w32.to(tokens.dtype), out.counts.long()
            self._last_logits, self.last_aux_loss, self.last_z_loss = out.logits, aux, z
            self.last_idx32, self.last_w32 = idx32, w32
            self._pending = dict(counts=out.counts, N=N, fused=True, events=out.events, z_loss=z.detach(),
                                 aux_loss=aux.detach(), elem=2, sram=16384 + ((E + 63) // 64) * 8192)
            return idx, w, counts
        # PyTorch path (bias, CPU, fp32 tokens, shapes the kernel does not cover): fp64 math under autograd
        logits64 = tokens.to(torch.float64) @ self.gate_w.to(torch.float64)
        if self.bias is not None:
            logits64 = logits64 + self.bias.to(torch.float64)
        probs = torch.softmax(logits64, dim=-1)
        vals, idx = torch.topk(probs, K, dim=-1, largest=True)
        w = (vals / vals.sum(-1, keepdim=True).clamp_min(1e-30)).to(tokens.dtype)
        counts = torch.bincount(idx.reshape(-1), minlength=E)
        f = counts.to(torch.float64) / float(N * K)
        self.last_aux_loss = (E * (f * probs.mean(0)).sum()).to(torch.float32)
        self.last_z_loss = (torch.logsumexp(logits64, dim=-1) ** 2).mean().to(torch.float32)
        self._last_logits = logits64.detach().to(tokens.dtype)
        self.last_idx32, self.last_w32 = idx.to(torch.int32), w.float()
        self._pending = dict(counts=counts, N=N, fused=False, events=None, z_loss=self.last_z_loss.detach(),
                             aux_loss=self.last_aux_loss.detach(), elem=tokens.element_size(), sram=0)
        return idx, w, counts
