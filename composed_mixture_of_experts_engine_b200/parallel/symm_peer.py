"""Peer-memory (NVLink P2P) transport of the expert-parallel MoE.

Per layer call, on one stream, with no host round trip:

    forward   publish x / idx / w in symmetric buffers            (local copies)
              barrier
              pull every rank's idx and w (a few hundred KB)       peer_allgather
              row plan of the local experts over all ranks' slots  moe_plan  (slot -> row table lands in symmetric memory)
              pull the rows that route here, expert-sorted         gather_rows_peer   <- the dispatch, P2P loads over NVLink
              grouped SwiGLU GEMMs (tcgen05); the epilogue of the second one copies every finished row out of its
              staging area straight into the buffer of the rank that owns the token (coalesced P2P stores that
              overlap the MMAs of later tiles)                          <- the combine transfer
              barrier
              y[t] = sum_k w * ycomb[t*K+k]                        combine_rows_peer on local rows
    backward  publish dy; barrier; d(gate) by dot products against the local ycomb rows; pull dy rows (scaled by
              the gate weights) inside the dgrad GEMM; the dX GEMM pushes its rows to the token owners; barrier;
              dx[t] = sum_k dxcomb[t*K+k]

``CMOE_EP_PUSH=0`` keeps the results on the expert's rank and lets the combine kernels pull them instead (measured
slower: 178.6 K against 188.6 K tokens/s on the two-GPU training benchmark); ``CMOE_EP_FUSED=0`` turns the dispatch
into a separate pull kernel.

Nothing is gathered that is not needed, nothing is reduced in bf16, and no buffer is materialised twice (the
library transport all-gathers x and reduce-scatters a [ep*T, H] partial result).  Barriers are flag words in
symmetric memory with a bounded wait; a peer that never arrives turns into a ``KernelTimeoutError`` at the next
``check_status``, not a hang.

Buffer reuse: x / idx / w / dy / dx staging buffers are shared by all layers (a barrier always separates the last
read of one use from the first write of the next); the result rows and the slot->row table live per layer
because the backward pass of the layer reads them again.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..ops import _ext
from ..ops import functional as OF
from ..ops import kernels
from . import symm
from .mesh import ParallelTopology

_FAILED: Optional[str] = None


def available(topology: Optional[ParallelTopology], axis: str) -> bool:
    if _FAILED is not None or not symm.enabled_for(topology, axis):
        return False
    return 1 < topology.axis_size(axis) <= 16


def _push() -> bool:
    """Result rows are pushed to the token owners by the GEMM epilogue (default) or pulled by the combine kernel (``CMOE_EP_PUSH=0``)."""
    return os.environ.get("CMOE_EP_PUSH", "1") != "0"


def _fused() -> bool:
    """Dispatch inside the grouped GEMM (default) or as a separate pull kernel (``CMOE_EP_FUSED=0``)."""
    return os.environ.get("CMOE_EP_FUSED", "1") != "0"


class _EPContext:
    """Symmetric buffers, flag words and the barrier epoch of one token-exchange group: the expert-parallel group
    (``axis="ep"``), or the expert-parallel x tensor-parallel block (``axis="etp"``) when the layer is handed
    sequence shards and every (expert, FFN slice) pair acts as an expert of its own."""

    def __init__(self, topo: ParallelTopology, axis: str = "ep"):
        self.topo = topo
        self.axis = axis
        self.slices = topo.tp_size if axis == "etp" else 1  # FFN slices per expert inside this group
        self.group = symm.group_for(topo, axis)
        self.rank, self.world = self.group.rank, self.group.world
        self.flags = self.group.flags
        self.flag_ptrs = self.flags.ptrs()
        self.epoch = 0
        self._shared: Dict[str, symm.SymmBuffer] = {}
        self._layer: Dict[tuple, symm.SymmBuffer] = {}
        self.expert_rank: Dict[int, torch.Tensor] = {}

    def barrier(self) -> None:
        self.epoch += 1
        _ext.ext().peer_barrier(self.flag_ptrs, self.rank, self.epoch, kernels.status_word(self.topo.device), 0)

    def shared(self, name: str, nbytes: int) -> symm.SymmBuffer:
        buf = self._shared.get(name)
        if buf is None or buf.local.numel() < nbytes:
            buf = self.group.alloc(f"ep.shared.{name}.{nbytes}", nbytes)
            self._shared[name] = buf
        return buf

    def per_layer(self, layer_key: int, name: str, nbytes: int) -> symm.SymmBuffer:
        key = (layer_key, name)
        buf = self._layer.get(key)
        if buf is None or buf.local.numel() < nbytes:
            buf = self.group.alloc(f"ep.layer{layer_key}.{name}.{nbytes}", nbytes)
            self._layer[key] = buf
        return buf

    def expert_rank_table(self, num_experts: int) -> torch.Tensor:
        """Group rank that owns each of the ``num_experts * slices`` exchange-level experts: expert ``g`` sliced
        ``j`` carries the id ``j * num_experts + g`` and lives on group rank ``owner(g) * slices + j``."""
        t = self.expert_rank.get(num_experts)
        if t is None:
            by_expert = []
            for r in range(self.topo.ep_size):
                by_expert += [r] * len(self.topo.experts_on_rank(num_experts, r))
            owner = [by_expert[g] * self.slices + j for j in range(self.slices) for g in range(num_experts)]
            t = torch.tensor(owner, dtype=torch.int32, device=self.topo.device)
            self.expert_rank[num_experts] = t
        return t


_CONTEXTS: Dict[tuple, _EPContext] = {}
_LAYER_KEYS: Dict[int, int] = {}


def _context(topo: ParallelTopology, axis: str = "ep") -> _EPContext:
    key = (axis,) + tuple(topo.axis_ranks(axis))
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = _EPContext(topo, axis)
        _CONTEXTS[key] = ctx
    return ctx


def _layer_key(layer) -> int:
    """Creation-ordered index of the layer (the same on every rank, which the collective allocations need)."""
    k = _LAYER_KEYS.get(id(layer))
    if k is None:
        k = len(_LAYER_KEYS)
        _LAYER_KEYS[id(layer)] = k
    return k


def _ptrs(buf: symm.SymmBuffer) -> List[int]:
    return buf.ptrs()


class _EPMoEPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate_w32, idx32, w13, w2, pc: _EPContext, lkey, expert_lo, num_experts, capacity,
                holder):
        # ``num_experts`` / ``expert_lo`` / ``idx32`` are exchange-level: with FFN slices as experts of their own
        # they count (expert, slice) pairs.  ``lkey`` = (layer, in-flight slot): the buffers that the backward
        # reads again exist once per microbatch that a pipeline stage can hold between forward and backward
        ext = _ext.ext()
        T, H = x.shape
        K = idx32.shape[1]
        ep, n_local = pc.world, w13.shape[0]
        dev = x.device
        cap_rows = kernels.ep_buffer_rows(T * K, n_local, ep * T * K)

        xs = pc.shared("x", T * H * 2)
        ids = pc.shared("idx", T * K * 4)
        ws = pc.shared("w", T * K * 4)
        xs.view(torch.bfloat16, T * H).view(T, H).copy_(x)
        ids.view(torch.int32, T * K).copy_(idx32.reshape(-1))
        ws.view(torch.float32, T * K).copy_(gate_w32.reshape(-1))
        pc.barrier()

        idx_all = torch.empty(ep * T, K, device=dev, dtype=torch.int32)
        w_all = torch.empty(ep * T, K, device=dev, dtype=torch.float32)
        ext.peer_allgather(_ptrs(ids), T * K * 4, idx_all)
        ext.peer_allgather(_ptrs(ws), T * K * 4, w_all)
        srow = pc.per_layer(lkey, "slot_row", ep * T * K * 4)
        plan = kernels.moe_plan(idx_all, num_experts, expert_lo=expert_lo, n_local=n_local, capacity=capacity * ep,
                                cap_rows=cap_rows, slot_row_out=srow.view(torch.int32, ep * T * K))
        xp = torch.empty(cap_rows, H, device=dev, dtype=torch.bfloat16)
        push = _push()
        erank = pc.expert_rank_table(num_experts // pc.slices)
        y = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        if push:
            ycs = pc.per_layer(lkey, "ycomb", T * K * H * 2)
            kw = dict(scatter=dict(row_slot=plan.row_slot, slots_per_rank=T * K, out_ptrs=_ptrs(ycs), out_ld=H))
        else:
            yps = pc.per_layer(lkey, "yp", cap_rows * H * 2)
            kw = dict(yp_out=yps.view(torch.bfloat16, cap_rows * H).view(cap_rows, H))
        if _fused():
            # the dispatch runs inside the first grouped GEMM: rows stream in over NVLink tile by tile
            kw["pull"] = dict(src_ptrs=_ptrs(xs), slots_per_src=T * K, pull_K=K, ld_src=H)
            if holder is not None and holder.get("want_stamps"):
                holder["pull_stamps"] = kernels.new_pull_stamps(dev)  # read back when telemetry is emitted
                kw["pull"]["stamps"] = holder["pull_stamps"]
        else:
            ext.gather_rows_peer(_ptrs(xs), T * K, K, plan.row_slot, None, xp, plan.num_m_tiles, H)
        hact, gu, _ = OF.grouped_swiglu_forward(xp, w13, w2, plan, **kw)
        pc.barrier()
        if push:
            ext.combine_rows_peer(_ptrs(ycs), _ptrs(srow), idx32, erank, gate_w32, y, K, pc.rank * T * K, H,
                                  ycs.view(torch.bfloat16, T * K * H).view(T * K, H))
        else:
            ext.combine_rows_peer(_ptrs(yps), _ptrs(srow), idx32, erank, gate_w32, y, K, pc.rank * T * K, H, None)
        ctx.push = push

        ctx.save_for_backward(xp, hact, gu, w_all, w13, w2, idx32, gate_w32)
        ctx.plan, ctx.pc, ctx.lkey, ctx.cap_rows = plan, pc, lkey, cap_rows
        ctx.num_experts = num_experts
        if holder is not None:
            holder["plan"] = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = _ext.ext()
        xp, hact, gu, w_all, w13, w2, idx32, gate_w32 = ctx.saved_tensors
        plan, pc, lkey, cap_rows = ctx.plan, ctx.pc, ctx.lkey, ctx.cap_rows
        T, K = idx32.shape
        H = xp.shape[1]
        dev = xp.device
        dy = dy.contiguous()
        dys = pc.shared("dy", T * H * 2)
        dys.view(torch.bfloat16, T * H).view(T, H).copy_(dy)
        pc.barrier()

        srow = pc.per_layer(lkey, "slot_row", pc.world * T * K * 4)
        erank = pc.expert_rank_table(ctx.num_experts // pc.slices)
        push = ctx.push
        slot_base = pc.rank * T * K
        d_gate = None
        if ctx.needs_input_grad[1]:
            d_gate = torch.empty(T, K, device=dev, dtype=torch.float32)
            if push:  # the forward left this rank's result rows here: no NVLink traffic
                ycs = pc.per_layer(lkey, "ycomb", T * K * H * 2)
                ext.combine_bwd_w_peer(_ptrs(ycs), _ptrs(srow), idx32, erank, dy, d_gate, K, slot_base, H,
                                       ycs.view(torch.bfloat16, T * K * H).view(T * K, H))
            else:
                yps = pc.per_layer(lkey, "yp", cap_rows * H * 2)
                ext.combine_bwd_w_peer(_ptrs(yps), _ptrs(srow), idx32, erank, dy, d_gate, K, slot_base, H, None)
        dyp = torch.empty(cap_rows, H, device=dev, dtype=torch.bfloat16)
        kw = {}
        if push:
            dxs = pc.shared("dxcomb", T * K * H * 2)
            kw["scatter"] = dict(row_slot=plan.row_slot, slots_per_rank=T * K, out_ptrs=_ptrs(dxs), out_ld=H)
        else:
            dxs = pc.shared("dxp", cap_rows * H * 2)
            kw["dxp_out"] = dxs.view(torch.bfloat16, cap_rows * H).view(cap_rows, H)
        if _fused():
            kw["pull"] = dict(src_ptrs=_ptrs(dys), slots_per_src=T * K, pull_K=K, ld_src=H,
                              slot_scale=w_all.reshape(-1))
        else:
            ext.gather_rows_peer(_ptrs(dys), T * K, K, plan.row_slot, w_all.reshape(-1), dyp, plan.num_m_tiles, H)
        need_dx = ctx.needs_input_grad[0]
        _, dw13, dw2 = OF.grouped_swiglu_backward(dyp, xp, hact, gu, w13, w2, plan, need_dx=need_dx, **kw)
        pc.barrier()
        dx = None
        if need_dx:
            dx = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
            local = dxs.view(torch.bfloat16, T * K * H).view(T * K, H) if push else None
            ext.combine_rows_peer(_ptrs(dxs), _ptrs(srow), idx32, erank, None, dx, K, slot_base, H, local)
        return dx, d_gate, None, dw13, dw2, None, None, None, None, None, None


def _in_flight_slot(layer) -> int:
    """Which of the layer's buffer sets this forward uses.  Under a 1F1B pipeline a stage runs up to ``pp`` forward
    passes of a layer before the first of their backward passes, so the tables and result rows that a backward pass
    reads again exist ``pp`` times and are handed out round-robin (backward passes run in forward order)."""
    n = max(1, layer.topology.pp_size)
    k = getattr(layer, "_peer_forward_calls", 0)
    layer._peer_forward_calls = k + 1
    return k % n if torch.is_grad_enabled() else n  # evaluation passes keep out of the training slots


def ep_moe(layer, flat: torch.Tensor, gate_w32: torch.Tensor, idx32: torch.Tensor, capacity: int, expert_lo: int
           ) -> torch.Tensor:
    global _FAILED
    try:
        pc = _context(layer.topology)
    except Exception as exc:  # symmetric memory could not be set up: all ranks fall back together
        _FAILED = f"{type(exc).__name__}: {exc}"
        raise
    with layer._timer.phase("experts"):
        return _EPMoEPeer.apply(flat, gate_w32, idx32, layer.w13, layer.w2, pc,
                                (_layer_key(layer), _in_flight_slot(layer)), expert_lo, layer.num_experts, capacity,
                                layer._last_plan_holder)


def ep_moe_sequence_shard(layer, shard: torch.Tensor, gate_w32: torch.Tensor, idx32: torch.Tensor, capacity: int,
                          expert_lo: int) -> torch.Tensor:
    """The layer under tensor + sequence parallelism, fed this rank's sequence shard ``shard`` [T_local, H] and its
    routing (``idx32`` / ``gate_w32`` [T_local, K]); returns the finished output rows of the same shard.

    Every (expert, FFN slice) pair is treated as an expert of its own: slice ``j`` of expert ``g`` gets the id
    ``j * E + g`` and lives on rank (owner(g), j) of the expert-parallel x tensor-parallel block.  A token routed to
    expert ``g`` is then routed to all ``tp`` slices of ``g`` with the same gate weight, and the weighted sum over
    its ``tp * K`` result rows is at once the top-k combine and the sum over the FFN slices.  With that, the
    sequence all-gather in front of the experts is the row pull inside the first grouped GEMM (each rank fetches the
    rows it needs from whichever rank holds that part of the sequence), and the reduce-scatter behind them is the
    row push of the second GEMM's epilogue followed by the local weighted sum: no separate collective, nothing
    replicated, and the router runs on the shard only."""
    global _FAILED
    topo = layer.topology
    try:
        pc = _context(topo, "etp")
    except Exception as exc:
        _FAILED = f"{type(exc).__name__}: {exc}"
        raise
    tp, E = topo.tp_size, layer.num_experts
    shift = torch.arange(tp, device=idx32.device, dtype=torch.int32).repeat_interleave(idx32.shape[1]) * E
    idx_eff = (idx32.repeat(1, tp) + shift[None, :]).contiguous()
    w_eff = gate_w32.repeat(1, tp)  # differentiable: the gradient of a gate weight sums over the slices
    with layer._timer.phase("experts"):
        return _EPMoEPeer.apply(shard, w_eff, idx_eff, layer.w13, layer.w2, pc,
                                (_layer_key(layer), _in_flight_slot(layer)), topo.tp_rank * E + expert_lo, E * tp,
                                capacity, layer._last_plan_holder)
