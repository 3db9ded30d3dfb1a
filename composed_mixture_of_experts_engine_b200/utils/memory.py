"""Per-GPU memory plan of a training configuration: what a rank holds and whether it fits a B200 (180 GB of HBM3e).

The trainer keeps whole bf16 parameters of the layers a rank owns (dense parameters replicated over data
parallelism, sliced by tensor and pipeline parallelism; experts additionally divided over expert parallelism), one
fp32 gradient buffer of the same extent (``main_grad``, which the weight-gradient GEMMs add into) and fp32 master weights plus two moments sharded over the ranks that hold the
same parameters (``ops/optim.py``).  Activations are estimated per micro-batch from the saved tensors of one decoder
block (sequence parallelism divides the norm / residual region by ``tp``).  The reference has no such planner.

    plan = plan_memory(cfg, world=8)
    print(format_plan(plan))
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

from .config import MoEConfig

__all__ = ["B200_HBM_GB", "parameter_counts", "plan_memory", "format_plan"]

B200_HBM_GB = 180.0
_GB = 1e9


def _attention_dims(cfg: MoEConfig):
    """(heads, kv heads, head width) of the decoder's attention; zeros for the attention-free toy model."""
    m = cfg.model
    if m.arch != "moe_decoder":
        return 0, 0, 0
    return m.resolved_num_heads, m.resolved_num_kv_heads, m.resolved_head_dim


def parameter_counts(cfg: MoEConfig) -> Dict[str, int]:
    """Parameter counts of the whole model by kind (no parallelism applied)."""
    m = cfg.model
    H, L, E, F, V = m.hidden_dim, m.num_layers, m.num_experts, m.ffn_dim, m.vocab_size
    heads, kv, hd = _attention_dims(cfg)
    attn = 0
    if heads:
        attn = L * (H * (heads + 2 * kv) * hd + heads * hd * H + H)  # wqkv, wo, attention norm
    experts = L * E * 3 * H * F
    router = L * H * E
    norms = L * H + H
    embed_head = 2 * V * H
    dense = attn + router + norms + embed_head
    return {"experts": experts, "attention": attn, "router": router, "norms": norms, "embed_and_head": embed_head,
            "dense": dense, "total": dense + experts,
            "active_per_token": dense - V * H + L * m.top_k * 3 * H * F}


def plan_memory(cfg: MoEConfig, world: Optional[int] = None, ep_buffer_factor: float = 1.5,
                mesh: Optional[Tuple[int, int, int, int, bool]] = None) -> Dict[str, float]:
    """Gigabytes per GPU by category for ``cfg`` on ``world`` ranks (default: the configured world size).
    ``mesh`` = (dp, ep, tp, pp, ep_from_dp) overrides the configured degrees (the trainer refits them to the
    number of ranks it was started with)."""
    par, m, t = cfg.parallelism, cfg.model, cfg.training
    if mesh is not None:
        dp, ep, tp, pp, ep_from_dp = mesh
        world = world or (dp * tp * pp if ep_from_dp else dp * ep * tp * pp)
    else:
        dp, ep, tp, pp = par.data_parallel, par.expert_parallel, par.tensor_parallel, par.pipeline_parallel
        ep_from_dp = bool(par.ep_from_dp)
        world = world or par.world_size
    counts = parameter_counts(cfg)
    # what one rank holds
    dense_local = counts["dense"] / (tp * pp)
    experts_local = counts["experts"] / (ep * tp * pp)
    # ranks that hold the same parameters (optimizer state is sharded over them)
    dense_replicas = dp if ep_from_dp else dp * ep
    expert_replicas = max(1, dp // ep) if ep_from_dp else dp
    weights = 2 * (dense_local + experts_local)
    grads = 4 * (dense_local + experts_local)
    optim = 12 * (dense_local / dense_replicas + experts_local / expert_replicas)
    # activations of one micro-batch, all blocks of this stage kept for the backward (no recomputation)
    S, H, F, K = m.sequence_length, m.hidden_dim, m.ffn_dim, m.top_k
    tokens = t.micro_batch_size * S
    layers_local = math.ceil(m.num_layers / pp)
    heads, kv, hd = _attention_dims(cfg)
    per_token_block = 2 * (2 * H / tp)  # residual stream + normed input (sequence-parallel region)
    if heads:
        per_token_block += 2 * ((heads + 2 * kv) * hd + heads * hd) / tp + 4 * heads / tp  # qkv, attention out, lse
    per_token_block += 2 * H + 2 * K * (H + 3 * F / tp) + K * 8  # MoE input, dispatched rows, gate|up, h, routing
    in_flight = min(pp, max(1, t.gradient_accumulation_steps)) if pp > 1 else 1
    activations = tokens * per_token_block * layers_local * in_flight
    logits = tokens * m.vocab_size * (2 + 4) / tp  # last stage: bf16 logits + fp32 softmax gradient
    ep_buffers = 0.0
    if ep > 1:
        rows = tokens * K * ep_buffer_factor
        ep_buffers = rows * (2 * H + 2 * 2 * F / tp + 2 * H)  # received rows, gate|up, outputs (symmetric memory)
    plan = {
        "world": world, "dp": dp, "ep": ep, "tp": tp, "pp": pp,
        "params_total_b": counts["total"] / 1e9, "params_active_b": counts["active_per_token"] / 1e9,
        "params_local_b": (dense_local + experts_local) / 1e9,
        "weights_gb": weights / _GB, "grads_gb": grads / _GB, "optimizer_gb": optim / _GB,
        "activations_gb": activations / _GB, "logits_gb": logits / _GB, "ep_buffers_gb": ep_buffers / _GB,
    }
    plan["total_gb"] = sum(v for k, v in plan.items() if k.endswith("_gb"))
    plan["hbm_gb"] = B200_HBM_GB
    plan["fits"] = plan["total_gb"] <= 0.92 * B200_HBM_GB  # allocator slack, NCCL / cuBLAS workspaces, CUDA context
    return plan


def format_plan(plan: Dict[str, float]) -> str:
    rows = [
        f"mesh dp{plan['dp']} x ep{plan['ep']} x tp{plan['tp']} x pp{plan['pp']} on {plan['world']} GPUs",
        f"parameters: {plan['params_total_b']:.2f} B total, {plan['params_active_b']:.2f} B active per token, "
        f"{plan['params_local_b']:.2f} B on this GPU",
    ]
    for key, label in (("weights_gb", "bf16 weights"), ("grads_gb", "gradient buffers"),
                       ("optimizer_gb", "fp32 master + moments (sharded)"), ("activations_gb", "activations"),
                       ("logits_gb", "logits + their gradient"), ("ep_buffers_gb", "expert-parallel row buffers")):
        rows.append(f"  {label:<34s} {plan[key]:8.1f} GB")
    verdict = "fits" if plan["fits"] else "DOES NOT FIT"
    rows.append(f"  {'total':<34s} {plan['total_gb']:8.1f} GB of {plan['hbm_gb']:.0f} GB: {verdict}")
    return "\n".join(rows)
