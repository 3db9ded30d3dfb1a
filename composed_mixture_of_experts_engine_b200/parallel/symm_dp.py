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


class DPPeer:
    """Peer-memory transport of one flat parameter group: its gradient and parameter buffers live in symmetric
    memory of the shard group, so that the reduce-scatter is one pull kernel (fp32 accumulation, cast and 1/world
    scale fused) and the parameter all-gather is one push kernel."""

    def __init__(self, topo, axis: str, name: str, numel: int, grad_dtype: torch.dtype):
        from ..ops import _ext, kernels

        self.sg = symm.group_for(topo, axis)
        self.rank, self.world = self.sg.rank, self.sg.world
        gbytes = numel * (2 if grad_dtype == torch.bfloat16 else 4)
        self.pbuf = self.sg.alloc(f"dp.{name}.params.{numel}", numel * 2)
        self.gbuf = self.sg.alloc(f"dp.{name}.grads.{numel}", gbytes)
        self.flat_p = self.pbuf.view(torch.bfloat16, numel)
        self.flat_g = self.gbuf.view(grad_dtype, numel)
        self.flat_p.zero_()
        self.flat_g.zero_()
        self.p_ptrs = self.pbuf.ptrs()
        self.g_ptrs = self.gbuf.ptrs()
        self.flag_ptrs = self.sg.flags.ptrs()
        self.device = topo.device
        self._ext, self._kernels = _ext, kernels

    def barrier(self) -> None:
        self.sg.epoch += 1
        self._ext.ext().peer_barrier(self.flag_ptrs, self.rank, self.sg.epoch, self._kernels.status_word(self.device), 0)

    def reduce_scatter(self, g, out: torch.Tensor) -> torch.Tensor:
        self.barrier()  # every rank has finished writing its gradients
        self._ext.ext().reduce_scatter_cast(self.g_ptrs, g.flat_g.dtype == torch.bfloat16, g.shard_lo, g.shard_numel,
                                            1.0 / self.world, out)
        self.barrier()  # every rank has finished reading: the gradient buffers may be cleared
        return out

    def all_gather(self, g) -> None:
        self._ext.ext().push_shard(self.p_ptrs, self.rank, g.shard_lo, g.shard_numel, g.flat_p)
        self.barrier()  # all shards have landed everywhere before the next forward reads the parameters


def make_peer(topo, axis: str, name: str, numel: int, grad_dtype: torch.dtype):
    """A :class:`DPPeer` when the peer-memory path is usable along ``axis``, else ``None`` (library collectives)."""
    import os

    if topo is None or os.environ.get("CMOE_DP_TRANSPORT", "auto") == "nccl":
        return None
    from . import symm_peer

    if not symm_peer.available(topo, axis):
        return None
    return DPPeer(topo, axis, name, numel, grad_dtype)
