"""Expert-parallel MoE on the device path: dropless, no host round trip, no count exchange.

Formulation.  With E experts spread over ``ep`` ranks, rank r evaluates its local experts on the tokens of ALL
ranks of its expert-parallel group and the per-token results are summed across ranks:

    forward    rows of x that route to a local expert are brought into the expert-sorted buffer xp
               -> grouped SwiGLU GEMMs (tcgen05) -> yp
               -> y[t] = sum_k w[t,k] * yp[owner(idx[t,k])][row(t,k)]
    backward   mirrored: dy rows in, weighted; grouped backward GEMMs; dx[t] = sum_k dxp[owner][row];
               d(gate)[t,k] = <dy[t], yp[owner][row]>

Every rank builds the row plan of its own experts from the routing decisions of all ranks (the indices are a
few KB per rank), so there is nothing to negotiate: no per-destination counts, no ``.item()``, no dynamic shapes
between ranks.  For top-k routing over ``ep`` ranks with k >= ep the bytes that cross NVLink equal those of a
dispatch/combine all-to-all (each token is needed by almost every rank anyway).

Transports (same math, chosen at run time):

* ``peer``: rows are pulled straight out of the peers' symmetric buffers by the gather / combine kernels
  (plain P2P loads over NVLink 5, bounded flag barriers between phases) - nothing is materialised twice.
* ``nccl``: all-gather of x (and of dy) + local gather, local combine into a partial result + reduce-scatter.
  This is the library baseline and the fallback when symmetric memory is unavailable.

Reference call sites replaced: C1-C3 of pkg/distributed/expert_parallel.py:104-218 and the expert loop /
scatter loop of pkg/distributed/moe_layer.py:318-353.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import kernels
from .mesh import ParallelTopology, ep_process_group


def _transport(layer) -> str:
    want = os.environ.get("CMOE_EP_TRANSPORT", "auto")
    if want in ("nccl", "peer"):
        return want
    from . import symm_peer

    return "peer" if symm_peer.available(layer.topology, "ep") else "nccl"


def _ag(t: torch.Tensor, group, ep: int) -> torch.Tensor:
    out = torch.empty((ep * t.shape[0],) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def _rs(t: torch.Tensor, group, ep: int) -> torch.Tensor:
    out = torch.empty((t.shape[0] // ep,) + tuple(t.shape[1:]), device=t.device, dtype=t.dtype)
    dist.reduce_scatter_tensor(out, t.contiguous(), group=group)
    return out


class _EPMoENccl(torch.autograd.Function):
    """Library transport: all-gather -> local expert FFN over all ranks' tokens -> reduce-scatter."""

    @staticmethod
    def forward(ctx, x, gate_w32, idx32, w13, w2, group, ep, expert_lo, num_experts, capacity, holder):
        n_local = w13.shape[0]
        x_all = _ag(x, group, ep)
        idx_all = _ag(idx32, group, ep)
        w_all = _ag(gate_w32, group, ep)
        T, K = idx32.shape
        # with capacity dropping the budget applies to the pooled tokens of the expert-parallel group
        # (ep x the per-rank capacity), first come first served in (rank, token) order
        plan = kernels.moe_plan(idx_all, num_experts, expert_lo=expert_lo, n_local=n_local, capacity=capacity * ep,
                                cap_rows=kernels.ep_buffer_rows(T * K, n_local, ep * T * K))
        xp = kernels.gather_rows(x_all, plan)
        del x_all
        hact, gu, yp = OF.grouped_swiglu_forward(xp, w13, w2, plan)
        y_part = kernels.combine_rows(yp, plan, w_all)
        y = _rs(y_part, group, ep)
        ctx.save_for_backward(xp, hact, gu, yp, w_all, w13, w2)
        ctx.plan, ctx.group, ctx.ep = plan, group, ep
        if holder is not None:
            holder["plan"] = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        xp, hact, gu, yp, w_all, w13, w2 = ctx.saved_tensors
        plan, group, ep = ctx.plan, ctx.group, ctx.ep
        dy_all = _ag(dy.contiguous(), group, ep)
        d_gate = None
        if ctx.needs_input_grad[1]:
            d_gate = _rs(kernels.combine_bwd_w(yp, plan, dy_all), group, ep)
        dyp = kernels.gather_rows(dy_all, plan, slot_scale=w_all.reshape(-1))
        del dy_all
        dxp, dw13, dw2 = OF.grouped_swiglu_backward(dyp, xp, hact, gu, w13, w2, plan,
                                                    need_dx=ctx.needs_input_grad[0])
        dx = None
        if dxp is not None:
            dx = _rs(kernels.combine_rows(dxp, plan, None), group, ep)
        return dx, d_gate, None, dw13, dw2, None, None, None, None, None, None


def moe_forward(layer, flat: torch.Tensor, gate_w32: torch.Tensor, idx32: torch.Tensor, capacity: int
                ) -> torch.Tensor:
    """Expert-parallel forward of ``layer`` for this rank's tokens ``flat`` [T, H] (bf16, CUDA)."""
    topo: ParallelTopology = layer.topology
    group = ep_process_group(topo)
    ep = topo.ep_size
    expert_lo = layer.local_expert_ids[0] if layer.local_expert_ids else 0
    gate_w32 = gate_w32.float().contiguous()
    idx32 = idx32.to(torch.int32).contiguous()
    if _transport(layer) == "peer":
        from . import symm_peer

        return symm_peer.ep_moe(layer, flat, gate_w32, idx32, capacity, expert_lo)
    with layer._timer.phase("experts"):
        return _EPMoENccl.apply(flat, gate_w32, idx32, layer.w13, layer.w2, group, ep, expert_lo, layer.num_experts,
                                capacity, layer._last_plan_holder)
