"""Data-parallel gradient reduce-scatter and parameter all-gather for the sharded optimizer.

``reduce_scatter_grads(group)`` returns this rank's fp32 shard of the gradient averaged over the shard
group; ``all_gather_params(group)`` makes the flat bf16 parameter buffer whole again after the shard was
updated.  Counterpart of FSDP2's collectives in the reference (pkg/distributed/data_parallel.py:74-97:
bf16 parameters, fp32 gradient reduction).

Library path: NCCL / gloo ``reduce_scatter_tensor`` on an fp32 copy and ``all_gather_into_tensor``.
Peer-memory path (CUDA, NVLink): one kernel reads every peer's bf16 gradient shard straight from its memory,
accumulates in fp32, scales by 1/world and writes the fp32 shard (reduce-scatter fused with cast and scale);
the parameter gather is a peer push of the updated bf16 shard.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import symm


def reduce_scatter_grads(g) -> torch.Tensor:
    world, group = g.shard_world, g.shard_group
    out = torch.empty(g.shard_numel, device=g.flat_g.device, dtype=torch.float32)
    peer = getattr(g, "peer", None)
    if peer is not None:
        return peer.reduce_scatter(g, out)
    full = g.flat_g if g.flat_g.dtype == torch.float32 else g.flat_g.float()
    if full.is_cuda:
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group)
    else:
        tmp = full.clone()
        dist.all_reduce(tmp, group=group)
        out.copy_(tmp[g.shard_lo:g.shard_lo + g.shard_numel])
    return out.div_(world)


def all_gather_params(g) -> None:
    peer = getattr(g, "peer", None)
    if peer is not None:
        peer.all_gather(g)
        return
    shard = g.flat_p[g.shard_lo:g.shard_lo + g.shard_numel]
    if g.flat_p.is_cuda:
        dist.all_gather_into_tensor(g.flat_p, shard.clone(), group=g.shard_group)
    else:
        parts = [torch.empty_like(shard) for _ in range(g.shard_world)]
        dist.all_gather(parts, shard.clone(), group=g.shard_group)
        g.flat_p.copy_(torch.cat(parts))
