"""``DistributedMoELayer``: top-k routed SwiGLU experts with expert / tensor parallelism.

Public surface of the reference layer (pkg/distributed/moe_layer.py:64-389): ``_cumcount``,
``compute_capacity_drop_mask``, ``_SwiGLUExpert`` and ``DistributedMoELayer`` with ``router``, ``experts``,
``local_expert_ids``, ``capacity_dropping`` and the ``last_*`` telemetry attributes.

What is computed is ``y_t = sum_k w[t,k] * Expert_{idx[t,k]}(x_t)`` with the expert chosen per (token, k)
slot.  (The reference sorts by ``idx[:,0]`` only and cuts the received rows into equal chunks,
``moe_layer.py:318-336``, so the expert applied there depends on row position; its multi-rank path also
sends counts that do not add up, ``:309-315``.)

Storage: the experts of this rank live in two stacked parameters, ``w13`` [E_local, 2F/tp, H] (gate rows,
then up rows) and ``w2`` [E_local, H, F/tp], which is what the grouped tcgen05 GEMMs consume.
``layer.experts[i]`` are views on those tensors with the reference's module structure
(``w_gate``/``w_up`` column-parallel, ``w_down`` row-parallel); replacing ``layer.experts`` with other
modules switches the layer to a generic per-expert loop.

Execution paths (chosen per call, same math):
  * CUDA + bf16, ep == 1: plan -> gather -> grouped GEMM (+SwiGLU epilogue) -> grouped GEMM -> combine.
  * CUDA + bf16, ep > 1 with NVLink peer memory: ``symm_ep`` (dispatch and combine inside the GEMM kernels).
  * anything else (CPU/gloo, fp32, no peer memory): autograd-aware all-to-all + PyTorch experts.
"""

from __future__ import annotations

import math
import weakref
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..ops.moe_router import MoERouter
from ..telemetry.logger import PhaseTimer
from . import collectives as C
from .mesh import ParallelTopology, ep_process_group, tp_process_group
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

__all__ = ["DistributedMoELayer", "_SwiGLUExpert", "compute_capacity_drop_mask", "_cumcount"]


# --------------------------------------------------------------------------------------------------
# capacity dropping (per k column, first come first served in token order)
# --------------------------------------------------------------------------------------------------
def _cumcount(idx: torch.Tensor) -> torch.Tensor:
    """For a 1-D tensor of ids: how many earlier positions hold the same id (0-based running count)."""
    if idx.numel() == 0:
        return torch.zeros_like(idx)
    order = torch.argsort(idx, stable=True)
    sorted_ids = idx[order]
    pos = torch.arange(idx.numel(), device=idx.device)
    is_start = torch.ones_like(sorted_ids, dtype=torch.bool)
    is_start[1:] = sorted_ids[1:] != sorted_ids[:-1]
    seg_start = torch.where(is_start, pos, torch.zeros_like(pos)).cummax(0).values
    out = torch.empty_like(idx)
    out[order] = (pos - seg_start).to(idx.dtype)
    return out


def compute_capacity_drop_mask(idx: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """Boolean [N, K]: True where the slot exceeds ``capacity`` tokens of its expert within its own k column."""
    if idx.dim() != 2:
        raise ValueError(f"idx must be [N, K], got {list(idx.shape)}")
    if capacity < 0:
        raise ValueError("capacity must be >= 0")
    cols = [_cumcount(idx[:, k]) >= capacity for k in range(idx.shape[1])]
    return torch.stack(cols, dim=1)


# --------------------------------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------------------------------
class _SwiGLUExpert(nn.Module):
    """``w_down(silu(w_gate(x)) * w_up(x))`` with the intermediate kept sharded over the tensor-parallel group."""

    def __init__(self, hidden_dim: int, ffn_dim: int, topology: Optional[ParallelTopology] = None,
                 dtype: Optional[torch.dtype] = None, device=None):
        super().__init__()
        hidden, ffn = hidden_dim, ffn_dim
        self.hidden, self.ffn = hidden, ffn
        self.w_gate = ColumnParallelLinear(hidden, ffn, bias=False, topology=topology, dtype=dtype, device=device,
                                           gather_output=False)
        self.w_up = ColumnParallelLinear(hidden, ffn, bias=False, topology=topology, dtype=dtype, device=device,
                                         gather_output=False)
        self.w_down = RowParallelLinear(ffn, hidden, bias=False, topology=topology, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w_down(F.silu(self.w_gate(x)) * self.w_up(x))


class _ViewLinearMixin:
    """A parallel linear whose ``weight`` is a live view into a stacked parameter of the owning layer."""

    def _bind(self, layer: "DistributedMoELayer", which: str, index: int) -> None:
        object.__setattr__(self, "_layer_ref", weakref.ref(layer))
        object.__setattr__(self, "_which", which)
        object.__setattr__(self, "_index", index)

    @property
    def weight(self) -> torch.Tensor:  # type: ignore[override]
        layer = self._layer_ref()
        f = layer.w13.shape[1] // 2
        if self._which == "gate":
            return layer.w13[self._index, :f]
        if self._which == "up":
            return layer.w13[self._index, f:]
        return layer.w2[self._index]

    @weight.setter
    def weight(self, value) -> None:
        if value is None:
            return
        with torch.no_grad():
            self.weight.copy_(value)


class _ViewColumn(_ViewLinearMixin, ColumnParallelLinear):
    def __init__(self, layer, which, index, in_f, out_f, topology):
        nn.Module.__init__(self)
        self.topology = topology
        self.tp_size = topology.tp_size if topology is not None else 1
        self.tp_rank = topology.tp_rank if topology is not None else 0
        self.in_features, self.out_features = in_f, out_f
        self.out_per_rank = out_f // self.tp_size
        self.gather_output, self.sequence_parallel, self.seq_dim = False, False, 1
        self.bias = None
        self._bind(layer, which, index)


class _ViewRow(_ViewLinearMixin, RowParallelLinear):
    def __init__(self, layer, index, in_f, out_f, topology):
        nn.Module.__init__(self)
        self.topology = topology
        self.tp_size = topology.tp_size if topology is not None else 1
        self.tp_rank = topology.tp_rank if topology is not None else 0
        self.in_features, self.out_features = in_f, out_f
        self.in_per_rank = in_f // self.tp_size
        self.sequence_parallel, self.seq_dim = False, 1
        self.bias = None
        self._bind(layer, "down", index)


class _ExpertView(_SwiGLUExpert):
    """Expert ``index`` of a layer's stacked weights, shaped like a ``_SwiGLUExpert`` (holds no parameters)."""

    def __init__(self, layer: "DistributedMoELayer", index: int, hidden: int, ffn: int, topology):
        nn.Module.__init__(self)
        self.hidden, self.ffn = hidden, ffn
        self.w_gate = _ViewColumn(layer, "gate", index, hidden, ffn, topology)
        self.w_up = _ViewColumn(layer, "up", index, hidden, ffn, topology)
        self.w_down = _ViewRow(layer, index, ffn, hidden, topology)


# --------------------------------------------------------------------------------------------------
# the layer
# --------------------------------------------------------------------------------------------------
class DistributedMoELayer(nn.Module):
    def __init__(self, hidden_dim: int, ffn_dim: int, num_experts: int, top_k: int,
                 topology: Optional[ParallelTopology] = None, capacity_factor: float = 1.25,
                 capacity_dropping: bool = False, dtype: torch.dtype = torch.float32, device=None,
                 init_std: Optional[float] = None):
        super().__init__()
        if topology is None:
            topology = ParallelTopology(1, 0, 1, 1)
        if not (1 <= top_k <= num_experts):
            raise ValueError(f"top_k ({top_k}) must be in [1, num_experts={num_experts}]")
        tp = topology.tp_size
        if ffn_dim % tp != 0:
            raise ValueError(f"ffn_dim ({ffn_dim}) must be divisible by tp_size ({tp})")
        self.hidden_dim, self.ffn_dim, self.num_experts, self.top_k = hidden_dim, ffn_dim, num_experts, top_k
        self.topology = topology
        self.capacity_factor = capacity_factor
        self.capacity_dropping = capacity_dropping
        self.local_expert_ids: List[int] = topology.experts_on_this_rank(num_experts)
        self.router = MoERouter(hidden_dim, num_experts, top_k, dtype=dtype)
        if device is not None:
            self.router.to(device)
        e_local, f_local = len(self.local_expert_ids), ffn_dim // tp
        self.w13 = nn.Parameter(torch.empty(max(e_local, 0), 2 * f_local, hidden_dim, dtype=dtype, device=device))
        self.w2 = nn.Parameter(torch.empty(max(e_local, 0), hidden_dim, f_local, dtype=dtype, device=device))
        self.w13.tensor_parallel_shard = self.w2.tensor_parallel_shard = True  # sliced on the FFN width over tp
        nn.init.normal_(self.w13, std=init_std if init_std is not None else 1.0 / math.sqrt(hidden_dim))
        nn.init.normal_(self.w2, std=init_std if init_std is not None else 1.0 / math.sqrt(ffn_dim))
        # the module list holds views only (no parameters), so state dicts and optimisers see w13 / w2 once
        self.experts = nn.ModuleList(
            [_ExpertView(self, i, hidden_dim, ffn_dim, topology) for i in range(e_local)])
        self._layer_id = id(self)
        self._timer = PhaseTimer(enabled=False)
        self._times = {}
        self._last_plan_holder: dict = {}
        self._last_n_slots = 0
        self._dropped_host: Optional[float] = 0.0
        self.force_library_path = False
        self.aux_scale = 1.0  # factor on this layer's router loss terms (1/tp when the router sees sequence shards)

    # ---- telemetry (resolved lazily: reading these waits for the recorded events only) ----------
    def enable_timing(self, on: bool = True) -> None:
        self._timer.enabled = on
        self._last_plan_holder["want_stamps"] = bool(on)  # fused dispatch: record device timestamps of the launch

    def _resolve(self) -> dict:
        got = self._timer.resolve(wait=True)
        if got:
            self._times = got
        return self._times

    @property
    def last_dispatch_ms(self) -> float:
        return float(self._resolve().get("dispatch", 0.0))

    @property
    def last_combine_ms(self) -> float:
        return float(self._resolve().get("combine", 0.0))

    @property
    def last_expert_compute_ms(self) -> float:
        return float(self._resolve().get("experts", 0.0))

    @property
    def last_overlap_ratio(self) -> float:
        """How much of the dispatch transfer ran under expert compute.  On the fused peer-memory path this comes
        from device timestamps inside the first grouped GEMM (first / last row pulled against first / last MMA of
        the same launch); on the library path from the event times of the dispatch and expert phases, as the
        reference does (pkg/distributed/moe_layer.py:340-341)."""
        stamps = self._last_plan_holder.get("pull_stamps")
        if stamps is not None:
            from ..ops.kernels import pull_overlap_ratio

            r = pull_overlap_ratio(stamps)
            if r is not None:
                return float(r)
        t = self._resolve()
        if "overlap_ratio" in t:
            return float(t["overlap_ratio"])
        d, c = t.get("dispatch", 0.0), t.get("experts", 0.0)
        return float(min(d / c, 1.0)) if c > 0 else 0.0

    @property
    def last_dropped_token_fraction(self) -> float:
        if self._dropped_host is not None:
            return self._dropped_host
        plan = self._last_plan_holder.get("plan")
        if plan is None or self._last_n_slots == 0:
            return 0.0
        kept = int(plan.counts_kept.sum().item())
        return max(0.0, 1.0 - kept / float(self._last_n_slots))

    # ---- helpers ----------------------------------------------------------------------------------
    def _experts_are_views(self) -> bool:
        return len(self.experts) == len(self.local_expert_ids) and all(isinstance(e, _ExpertView) for e in self.experts)

    def _expert_to_rank(self, expert_id):
        """EP rank that owns ``expert_id`` (contiguous blocks, remainder on the lowest ranks).  Takes an int and
        returns an int, or takes an integer tensor of any shape and returns a tensor of ranks of that shape
        (reference: pkg/distributed/moe_layer.py:362-389)."""
        ep = self.topology.ep_size
        per, rem = divmod(self.num_experts, ep)
        boundary = rem * (per + 1)
        if torch.is_tensor(expert_id):
            e = expert_id.long()
            low = torch.div(e, per + 1, rounding_mode="floor")
            high = rem + torch.div(e - boundary, max(per, 1), rounding_mode="floor")
            return torch.where(e < boundary, low, high)
        if expert_id < boundary:
            return expert_id // (per + 1)
        return rem + (expert_id - boundary) // max(per, 1)

    def capacity(self, n_tokens: int) -> int:
        return math.ceil(self.capacity_factor * n_tokens * self.top_k / self.num_experts)

    # ---- forward ----------------------------------------------------------------------------------
    def fused_sequence_shard_path(self, tokens: torch.Tensor) -> bool:
        """True when the layer can take this rank's sequence shard directly under tensor + sequence parallelism:
        CUDA bf16 tensors and peer memory over the expert-parallel x tensor-parallel block.  The gather of the
        sequence and the reduce-scatter of the result then happen inside the grouped GEMM kernels
        (``symm_peer.ep_moe_sequence_shard``) instead of as collectives around the layer."""
        topo = self.topology
        if topo.tp_size <= 1 or not dist.is_initialized() or self.force_library_path:
            return False
        if not (OF.on_device_path(tokens, self.w13, self.w2) and self._experts_are_views()):
            return False
        import os

        if os.environ.get("CMOE_EP_TRANSPORT", "auto") == "nccl":
            return False
        from . import symm_peer

        return symm_peer.available(topo, "etp")

    def _forward_sequence_shard(self, tokens: torch.Tensor) -> torch.Tensor:
        flat = tokens.reshape(-1, tokens.shape[-1])
        topo = self.topology
        # the router sees this rank's part of the sequence only: its gate gradient and its loss terms are partial
        # sums over the tensor-parallel group (summed after the backward pass, like the norm weights' gradients)
        self.router.gate_w.sequence_parallel_grad = True
        self.aux_scale = 1.0 / topo.tp_size
        idx, _w, _counts = self.router(flat)
        gate_w = self.router.last_w32
        N = flat.shape[0]
        cap = self.capacity(N) if self.capacity_dropping else 0
        self._last_n_slots = N * self.top_k * topo.tp_size
        self._dropped_host = None if cap > 0 else 0.0
        idx32 = self.router.last_idx32 if self.router.last_idx32 is not None else idx.to(torch.int32)
        from . import symm_peer

        expert_lo = self.local_expert_ids[0] if self.local_expert_ids else 0
        y = symm_peer.ep_moe_sequence_shard(self, flat.contiguous(), gate_w.float().contiguous(),
                                            idx32.to(torch.int32).contiguous(), cap, expert_lo)
        return y.reshape(tokens.shape)

    def forward(self, tokens: torch.Tensor, sequence_shard: bool = False) -> torch.Tensor:
        """``sequence_shard=True``: ``tokens`` is this rank's shard of a sequence that is split over the
        tensor-parallel group and the result is the same shard of the output (only where
        :meth:`fused_sequence_shard_path` holds); otherwise every tensor-parallel rank passes the same tokens."""
        if sequence_shard:
            return self._forward_sequence_shard(tokens)
        if tokens.dim() == 3:
            B, S, H = tokens.shape
            flat = tokens.reshape(B * S, H)
        elif tokens.dim() == 2:
            flat = tokens
        else:
            raise ValueError(f"DistributedMoELayer expects [B,S,H] or [N,H], got shape {list(tokens.shape)}")
        if flat.shape[-1] != self.hidden_dim:
            raise ValueError(f"hidden size {flat.shape[-1]} != layer hidden_dim {self.hidden_dim}")
        topo = self.topology
        N = flat.shape[0]
        idx, w, _counts = self.router(flat)
        gate_w = self.router.last_w32  # fp32 gate weights, differentiable on every path
        if topo.tp_size > 1:
            # The router runs replicated on every tensor-parallel rank; the experts are sliced on the FFN width, so
            # each rank produces partial sums.  Their gradients with respect to the tokens AND to the gate weights
            # are partial too: both enter the sliced region through an identity whose backward is an all-reduce.
            flat = C.copy_to_group(flat, tp_process_group(topo))
            gate_w = C.copy_to_group(gate_w, tp_process_group(topo))
        cap = self.capacity(N) if self.capacity_dropping else 0
        self._last_n_slots = N * self.top_k

        device_path = (OF.on_device_path(flat, self.w13, self.w2) and self._experts_are_views()
                       and not self.force_library_path)
        ep_active = topo.ep_size > 1 and dist.is_initialized()
        if device_path and not ep_active:
            self._dropped_host = None if cap > 0 else 0.0
            idx32 = self.router.last_idx32 if self.router.last_idx32 is not None else idx.to(torch.int32)
            with self._timer.phase("experts"):
                y = OF.local_moe(flat, gate_w, idx32, self.w13, self.w2, cap, self._last_plan_holder)
        elif device_path and ep_active:
            from . import symm_ep

            self._dropped_host = None if cap > 0 else 0.0
            idx32 = self.router.last_idx32 if self.router.last_idx32 is not None else idx.to(torch.int32)
            y = symm_ep.moe_forward(self, flat, gate_w, idx32, cap)
        else:
            y = self._library_forward(flat, idx, gate_w, cap)

        if topo.tp_size > 1:
            y = C.all_reduce(y, tp_process_group(topo))
        return y.reshape(tokens.shape)

    def _peer_path_ok(self) -> bool:
        from . import symm

        return symm.enabled_for(self.topology, "ep")

    # ---- library path: autograd-aware all-to-all + PyTorch experts --------------------------------
    def _run_local_experts(self, rows: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """``rows`` grouped by local expert with ``counts[i]`` rows each."""
        outs, start = [], 0
        views = self._experts_are_views()
        f = self.w13.shape[1] // 2
        for i, c in enumerate(counts):
            if c == 0:
                continue
            seg = rows[start:start + c]
            if views:
                g = seg @ self.w13[i, :f].t()
                u = seg @ self.w13[i, f:].t()
                outs.append((F.silu(g) * u) @ self.w2[i].t())
            else:
                outs.append(self.experts[i](seg))
            start += c
        if not outs:
            return rows.new_zeros(0, self.hidden_dim)
        return torch.cat(outs, dim=0)

    def _library_forward(self, flat: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, cap: int) -> torch.Tensor:
        topo = self.topology
        N, K, E = flat.shape[0], self.top_k, self.num_experts
        ep = topo.ep_size if dist.is_initialized() else 1
        flat_e = idx.reshape(-1)
        if cap > 0:
            drop = compute_capacity_drop_mask(idx, E, cap).reshape(-1)
            self._dropped_host = float(drop.float().mean().item())
            flat_e = torch.where(drop, torch.full_like(flat_e, E), flat_e)
        else:
            self._dropped_host = 0.0
        order = torch.argsort(flat_e, stable=True)
        cnt_e = torch.bincount(flat_e, minlength=E + 1)[:E]
        n_kept = int(cnt_e.sum().item())
        order = order[:n_kept]
        tok_of = torch.div(order, K, rounding_mode="floor")
        rows = flat.index_select(0, tok_of)
        w_rows = w.reshape(-1).index_select(0, order)

        if ep == 1:
            with self._timer.phase("experts"):
                out_rows = self._run_local_experts(rows, [int(c) for c in cnt_e.tolist()])
        else:
            group = ep_process_group(topo)
            max_local = -(-E // ep)
            owners = [topo.experts_on_rank(E, r) for r in range(ep)]
            cnt_list = [int(c) for c in cnt_e.tolist()]
            send_counts = [sum(cnt_list[e] for e in owners[r]) for r in range(ep)]
            table = torch.zeros(ep, max_local, dtype=torch.int64, device=flat.device)
            for r in range(ep):
                for j, e in enumerate(owners[r]):
                    table[r, j] = cnt_list[e]
            recv_table = C.exchange_counts(table, group).tolist()  # [src][local expert]
            recv_counts = [int(sum(row)) for row in recv_table]
            with self._timer.phase("dispatch"):
                received = C.all_to_all_rows(rows, send_counts, recv_counts, group)
            n_local = len(self.local_expert_ids)
            # received is ordered (source, expert); regroup to (expert, source)
            src_off = [0]
            for c in recv_counts:
                src_off.append(src_off[-1] + c)
            perm_parts, per_expert = [], []
            for j in range(n_local):
                tot = 0
                for s in range(ep):
                    start = src_off[s] + int(sum(recv_table[s][:j]))
                    c = int(recv_table[s][j])
                    if c:
                        perm_parts.append(torch.arange(start, start + c, device=flat.device))
                    tot += c
                per_expert.append(tot)
            perm = torch.cat(perm_parts) if perm_parts else torch.zeros(0, dtype=torch.long, device=flat.device)
            with self._timer.phase("experts"):
                out_grouped = self._run_local_experts(received.index_select(0, perm), per_expert)
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel(), device=flat.device)
            expert_out = out_grouped.index_select(0, inv) if perm.numel() else received.new_zeros(0, self.hidden_dim)
            with self._timer.phase("combine"):
                out_rows = C.all_to_all_rows(expert_out, recv_counts, send_counts, group)

        y = torch.zeros(N, self.hidden_dim, dtype=torch.float32, device=flat.device)
        y = y.index_add(0, tok_of, out_rows.float() * w_rows.float()[:, None])
        return y.to(flat.dtype)
