"""Autograd-aware collectives over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

The reference calls raw ``dist.*`` into ``torch.empty`` buffers, so no gradient ever crosses a
tensor- or expert-parallel boundary (pkg/distributed/expert_parallel.py:109-113,
tensor_parallel.py:123-128).  Each function here defines its backward as the transposed collective:
all-gather <-> reduce-scatter, all-reduce <-> identity, all-to-all <-> reversed all-to-all.
These are the library path (CPU runs, the multi-rank oracle, and the comparator of the fused
peer-memory kernels); the fused sm_100a paths replace them where they apply.
"""

from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


def _size(group) -> int:
    return dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1


def _all_gather_cat(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    xc = x.contiguous()
    parts = [torch.empty_like(xc) for _ in range(n)]
    dist.all_gather(parts, xc, group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    rank = dist.get_rank(group)
    chunks = [c.contiguous() for c in x.chunk(n, dim=dim)]
    if x.is_cuda:
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=group)
        return out
    # gloo has no reduce-scatter: all-reduce and keep this rank's slice
    full = x.contiguous().clone()
    dist.all_reduce(full, group=group)
    return full.chunk(n, dim=dim)[rank].contiguous()


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group, rs_grad):
        ctx.dim, ctx.group, ctx.rs_grad = dim, group, rs_grad
        return _all_gather_cat(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.rs_grad:
            return _reduce_scatter_dim(g, ctx.dim, ctx.group), None, None, None
        n = _size(ctx.group)
        if n == 1:
            return g, None, None, None
        return g.chunk(n, dim=ctx.dim)[dist.get_rank(ctx.group)].contiguous(), None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _reduce_scatter_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_cat(g, ctx.dim, ctx.group), None, None


class _AllReduce(torch.autograd.Function):
    """Forward all-reduce(sum), backward identity (the gradient of a replicated consumer is already whole)."""

    @staticmethod
    def forward(ctx, x, group):
        if _size(group) == 1:
            return x
        out = x.contiguous().clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToGroup(torch.autograd.Function):
    """Forward identity, backward all-reduce(sum): entry of a region whose input is replicated."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if _size(ctx.group) == 1:
            return g, None
        out = g.contiguous().clone()
        dist.all_reduce(out, group=ctx.group)
        return out, None


class _Split(torch.autograd.Function):
    """Forward: keep this rank's chunk along ``dim``; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        n = _size(group)
        if n == 1:
            return x
        return x.chunk(n, dim=dim)[dist.get_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_cat(g, ctx.dim, ctx.group), None, None


def _all_to_all_rows(x: torch.Tensor, send: List[int], recv: List[int], group) -> torch.Tensor:
    out = torch.empty((sum(recv),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
    return out


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        return _all_to_all_rows(x, send, recv, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all_rows(g, ctx.recv, ctx.send, ctx.group), None, None, None


def all_gather(x: torch.Tensor, dim: int, group, reduce_scatter_grad: bool = True) -> torch.Tensor:
    return x if _size(group) == 1 else _AllGather.apply(x, dim, group, reduce_scatter_grad)


def reduce_scatter(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    return x if _size(group) == 1 else _ReduceScatter.apply(x, dim, group)


def all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    return x if _size(group) == 1 else _AllReduce.apply(x, group)


def copy_to_group(x: torch.Tensor, group) -> torch.Tensor:
    return x if _size(group) == 1 else _CopyToGroup.apply(x, group)


def split(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    return x if _size(group) == 1 else _Split.apply(x, dim, group)


def all_to_all_rows(x: torch.Tensor, send_counts: List[int], recv_counts: List[int], group) -> torch.Tensor:
    """Uneven all-to-all of rows: ``send_counts[r]`` rows go to rank r, ``recv_counts[r]`` rows arrive from it."""
    if _size(group) == 1:
        return x
    return _AllToAllRows.apply(x, list(send_counts), list(recv_counts), group)


def exchange_counts(counts: torch.Tensor, group) -> torch.Tensor:
    """counts[r, ...] is what this rank sends to rank r; returns what each rank sends to this one."""
    if _size(group) == 1:
        return counts
    out = torch.empty_like(counts)
    dist.all_to_all_single(out, counts.contiguous(), group=group)
    return out
