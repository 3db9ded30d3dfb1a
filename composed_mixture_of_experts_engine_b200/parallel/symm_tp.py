"""Peer-memory path of the sequence-parallel tensor-parallel linears (CUDA, bf16, NVLink).

``allgather_linear``: every rank publishes its sequence shard in a symmetric buffer; after one bounded barrier the
GEMM kernel itself pulls the rows of all shards (four extra warps per CTA, plain P2P loads) while its tensor-core
pipeline consumes the tiles that have landed, so the all-gather overlaps the GEMM tile by tile and the gathered
activation is written exactly once (it is also what the weight gradient needs later).

``linear_reduce_scatter``: the GEMM's epilogue stores every partial result row straight into a staging slab on the
rank that owns that sequence position (plain P2P stores, so the scatter overlaps the MMAs of later tiles); after
one barrier each rank sums the ``tp`` slabs it received in fp32 from its own memory.  ``CMOE_TP_PUSH=0`` keeps the
partial result local and lets each rank pull and sum the rows of its shard instead.

Both are differentiable; the backward of one is the forward pattern of the other.  Replaces call sites C4-C7
(pkg/distributed/tensor_parallel.py:128,201-206; sequence_parallel.py:131,165).
"""

from __future__ import annotations

import os
from typing import Dict, List, Tuple

import torch

from ..ops import _ext, kernels
from ..ops.kernels import EPI_STORE, MoEPlan
from . import symm
from .mesh import ParallelTopology


class _TPContext:
    def __init__(self, topo: ParallelTopology):
        self.topo = topo
        self.sg = symm.group_for(topo, "tp")
        self.rank, self.world = self.sg.rank, self.sg.world
        self.flag_ptrs = self.sg.flags.ptrs()
        self._bufs: Dict[str, symm.SymmBuffer] = {}
        self._plans: Dict[Tuple[int, int], Tuple[MoEPlan, torch.Tensor]] = {}
        self._scatter: Dict[Tuple[int, int], Tuple[torch.Tensor, int, torch.Tensor]] = {}

    def barrier(self) -> None:
        self.sg.epoch += 1
        _ext.ext().peer_barrier(self.flag_ptrs, self.rank, self.sg.epoch, kernels.status_word(self.topo.device), 0)

    def buf(self, name: str, nbytes: int) -> symm.SymmBuffer:
        b = self._bufs.get(name)
        if b is None or b.local.numel() < nbytes:
            b = self.sg.alloc(f"tp.{name}.{nbytes}", nbytes)
            self._bufs[name] = b
        return b

    def gather_plan(self, batch: int, s_local: int) -> Tuple[MoEPlan, torch.Tensor]:
        """Row plan of the gathered activation [batch * tp * s_local rows]: full row (b, r, s) comes from row
        b * s_local + s of rank r.  Also returns the map from this rank's shard rows to full rows."""
        key = (batch, s_local)
        hit = self._plans.get(key)
        if hit is not None:
            return hit
        dev, tp = self.topo.device, self.world
        rows = batch * tp * s_local
        cap = (rows + 127) // 128 * 128
        b = torch.arange(batch, device=dev).view(batch, 1, 1)
        r = torch.arange(tp, device=dev).view(1, tp, 1)
        s = torch.arange(s_local, device=dev).view(1, 1, s_local)
        slot = (r * (batch * s_local) + b * s_local + s).reshape(-1).to(torch.int32)
        plan = MoEPlan(rows, 1, 1, cap, dev)
        plan.row_slot.fill_(-1)
        plan.row_slot[:rows] = slot
        plan.tile_group.zero_()
        plan.num_m_tiles.fill_(cap // 128)
        own = (b * (tp * s_local) + self.rank * s_local + s).expand(batch, 1, s_local).reshape(-1).to(torch.int32)
        self._plans[key] = (plan, own.contiguous())
        return self._plans[key]

    def scatter_plan(self, batch: int, s_local: int) -> Tuple[torch.Tensor, int, torch.Tensor]:
        """(row slots [batch*tp*s_local], slots per rank, identity row map [batch*s_local]): full row (b, r, s) of this
        rank's partial result goes to rank r, row  rank * batch*s_local + b*s_local + s  of its staging buffer; as a
        slot number that is  r * slots_per_rank + row."""
        key = (batch, s_local)
        hit = self._scatter.get(key)
        if hit is None:
            dev, tp = self.topo.device, self.world
            per_rank = tp * batch * s_local
            b = torch.arange(batch, device=dev).view(batch, 1, 1)
            r = torch.arange(tp, device=dev).view(1, tp, 1)
            s = torch.arange(s_local, device=dev).view(1, 1, s_local)
            slot = r * per_rank + self.rank * (batch * s_local) + b * s_local + s
            hit = (slot.reshape(-1).to(torch.int32).contiguous(), per_rank,
                   torch.arange(batch * s_local, device=dev, dtype=torch.int32))
            self._scatter[key] = hit
        return hit


_CTX: Dict[tuple, _TPContext] = {}


def _ctx(topo: ParallelTopology) -> _TPContext:
    key = tuple(topo.axis_ranks("tp"))
    if key not in _CTX:
        _CTX[key] = _TPContext(topo)
    return _CTX[key]


def _ptrs(buf: symm.SymmBuffer) -> List[int]:
    return buf.ptrs()


def _gathered_gemm(c: _TPContext, shard2d: torch.Tensor, weight: torch.Tensor, batch: int, s_local: int,
                   b_mn: bool, name: str):
    """(full activation [rows, K], out [rows, N]) with the gather running inside the GEMM kernel."""
    rows_local, Kdim = shard2d.shape
    N = weight.shape[1] if b_mn else weight.shape[0]
    plan, _ = c.gather_plan(batch, s_local)
    xs = c.buf(name, rows_local * Kdim * 2)
    xs.view(torch.bfloat16, rows_local * Kdim).view(rows_local, Kdim).copy_(shard2d)
    c.barrier()
    full = torch.empty(plan.cap_rows, Kdim, device=shard2d.device, dtype=torch.bfloat16)
    out = torch.empty(plan.cap_rows, N, device=shard2d.device, dtype=torch.bfloat16)
    kernels.gemm_pull(full, weight, out, plan, epilogue=EPI_STORE, N=N, K=Kdim, groups=1, b_group_rows=0, b_mn=b_mn,
                      src_ptrs=_ptrs(xs), slots_per_src=rows_local, pull_K=1, ld_src=Kdim)
    c.barrier()  # the shard buffer may be overwritten by the next call once everybody has pulled
    rows = batch * c.world * s_local
    return full[:rows], out[:rows]


def _reduce_scattered(c: _TPContext, part: torch.Tensor, batch: int, s_local: int, name: str) -> torch.Tensor:
    """This rank's sequence shard of the sum over ranks of ``part`` [batch * tp * s_local, N] (in symmetric memory)."""
    _, own = c.gather_plan(batch, s_local)
    N = part.shape[1]
    c.barrier()
    out = torch.empty(batch * s_local, N, device=part.device, dtype=torch.bfloat16)
    buf = c.buf(name, part.numel() * 2)
    _ext.ext().reduce_rows_peer(_ptrs(buf), own, out, N)
    c.barrier()
    return out


def _partial_gemm(c: _TPContext, x2d: torch.Tensor, weight: torch.Tensor, b_mn: bool, name: str) -> torch.Tensor:
    rows = x2d.shape[0]
    N = weight.shape[1] if b_mn else weight.shape[0]
    buf = c.buf(name, rows * N * 2)
    part = buf.view(torch.bfloat16, rows * N).view(rows, N)
    kernels.gemm(x2d, weight, part, M=rows, N=N, K=x2d.shape[1], b_mn=b_mn)
    return part


def _push() -> bool:
    return os.environ.get("CMOE_TP_PUSH", "1") != "0"


def _gemm_reduce_scatter(c: _TPContext, x2d: torch.Tensor, weight: torch.Tensor, b_mn: bool, batch: int,
                         s_local: int, name: str) -> torch.Tensor:
    """Sequence shard of  sum over ranks of (x2d @ W)  with the scatter fused into the GEMM epilogue."""
    if not _push():
        return _reduce_scattered(c, _partial_gemm(c, x2d, weight, b_mn, name), batch, s_local, name)
    rows = x2d.shape[0]
    N = weight.shape[1] if b_mn else weight.shape[0]
    shard_rows = batch * s_local
    slots, per_rank, ident = c.scatter_plan(batch, s_local)
    stage = c.buf(name + ".stage", c.world * shard_rows * N * 2)
    c.barrier()  # every rank has finished reading its slabs of the previous call
    kernels.gemm_scatter(x2d, weight, N=N, K=x2d.shape[1], row_slot=slots, slots_per_rank=per_rank,
                         out_ptrs=_ptrs(stage), out_ld=N, b_mn=b_mn, M=rows)
    c.barrier()
    out = torch.empty(shard_rows, N, device=x2d.device, dtype=torch.bfloat16)
    base = stage.local.data_ptr()
    slabs = [base + j * shard_rows * N * 2 for j in range(c.world)]  # all local: the partial sums are already here
    _ext.ext().reduce_rows_peer(slabs, ident, out, N)
    return out


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, c: _TPContext):
        B, S_l, Kdim = x.shape
        full, out = _gathered_gemm(c, x.reshape(B * S_l, Kdim), weight, B, S_l, False, "ag_x")
        ctx.save_for_backward(full, weight)
        ctx.c, ctx.dims = c, (B, S_l)
        return out.view(B, c.world * S_l, weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        full, weight = ctx.saved_tensors
        c, (B, S_l) = ctx.c, ctx.dims
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            # dy [rows, out_l] @ W [out_l, in], summed over ranks, this rank's sequence shard
            dx = _gemm_reduce_scatter(c, dy2, weight, True, B, S_l, "ag_dx").view(B, S_l, -1)
        dw = kernels.linear_tn(dy2, full).to(weight.dtype) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, c: _TPContext):
        B, S, Kdim = x.shape
        S_l = S // c.world
        x2 = x.reshape(B * S, Kdim).contiguous()
        y = _gemm_reduce_scatter(c, x2, weight, False, B, S_l, "rs_y")
        ctx.save_for_backward(x2, weight)
        ctx.c, ctx.dims = c, (B, S_l)
        return y.view(B, S_l, weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        c, (B, S_l) = ctx.c, ctx.dims
        dy_full, dx = _gathered_gemm(c, dy.reshape(B * S_l, -1).contiguous(), weight, B, S_l, True, "rs_dy")
        dw = kernels.linear_tn(dy_full.contiguous(), x2).to(weight.dtype) if ctx.needs_input_grad[1] else None
        return dx.reshape(B, c.world * S_l, -1) if ctx.needs_input_grad[0] else None, dw, None


def allgather_linear(x: torch.Tensor, w: torch.Tensor, topo: ParallelTopology, seq_dim: int = 1) -> torch.Tensor:
    if x.dim() != 3 or seq_dim != 1:
        raise ValueError("the peer path expects [batch, seq/tp, features] with the sequence on dim 1")
    return _AllGatherLinear.apply(x, w, _ctx(topo))


def linear_reduce_scatter(x: torch.Tensor, w: torch.Tensor, topo: ParallelTopology, seq_dim: int = 1) -> torch.Tensor:
    if x.dim() != 3 or seq_dim != 1:
        raise ValueError("the peer path expects [batch, seq, features/tp] with the sequence on dim 1")
    return _LinearReduceScatter.apply(x, w, _ctx(topo))
