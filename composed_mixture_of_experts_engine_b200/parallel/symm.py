"""Symmetric (peer-mapped) memory for the fused compute+collective kernels.

One :class:`SymmGroup` per process group: buffers are allocated with ``torch.distributed._symmetric_memory``
(CUDA virtual memory mapped into every peer of the group over NVLink), and what the kernels receive is a
small device table of the peers' base addresses.  Nothing here launches a kernel that waits without a bound.

The reference has no counterpart: it only calls NCCL / gloo collectives (call sites:
pkg/distributed/expert_parallel.py:104-218, tensor_parallel.py:128,201).
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import debug

from .mesh import ParallelTopology, dp_process_group, ep_process_group, tp_process_group

_GROUPS: Dict[Tuple[str, Tuple[int, ...]], "SymmGroup"] = {}
_DISABLED_REASON: Optional[str] = None


def _axis_group(topo: ParallelTopology, axis: str):
    from .mesh import ddp_process_group, edp_process_group, etp_process_group

    return {"ep": ep_process_group, "tp": tp_process_group, "dp": dp_process_group,
            "edp": edp_process_group, "ddp": ddp_process_group, "etp": etp_process_group}[axis](topo)


def enabled_for(topo: Optional[ParallelTopology], axis: str) -> bool:
    """True when the fused peer-memory kernels may be used along ``axis`` of this topology."""
    if topo is None or not dist.is_initialized() or not torch.cuda.is_available():
        return False
    if os.environ.get("CMOE_DISABLE_PEER_KERNELS", "0") == "1" or _DISABLED_REASON is not None:
        return False
    size = topo.axis_size(axis)
    if size <= 1 or topo.device.type != "cuda":
        return False
    if dist.get_backend() != "nccl":
        return False
    return True


class SymmBuffer:
    """A buffer that exists at the same size on every rank of a group, with all peers' addresses.

    ``local`` is this rank's usable part; ``ptrs()`` are the addresses of the same part on every rank.  With
    ``CMOE_DEBUG_BOUNDS=1`` the allocation carries a guard band on either side (``guard``), which
    ``SymmGroup.verify_guards`` checks: a peer kernel that wrote outside its buffer shows up there."""

    def __init__(self, full: torch.Tensor, handle, world: int, nbytes: int, guard=None):
        self.full = full
        self.handle = handle
        self.guard = guard
        self.offset = debug.GUARD_BYTES if guard is not None else 0
        self.local = full[self.offset:self.offset + nbytes]
        self.world = world

    def ptrs(self):
        return [int(p) + self.offset for p in self.handle.buffer_ptrs]

    def view(self, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        raw = self.local.view(torch.uint8)[offset_bytes:offset_bytes + numel * torch.empty((), dtype=dtype).element_size()]
        return raw.view(dtype)


class SymmGroup:
    def __init__(self, group, ranks: Tuple[int, ...], device: torch.device):
        self.group, self.ranks, self.device = group, ranks, device
        self.world = len(ranks)
        self.rank = dist.get_rank(group)
        self._buffers: Dict[str, SymmBuffer] = {}
        self.epoch = 0
        # flag words: [0, world) barrier arrivals; the rest is handed out to kernels by name
        self.flags = self.alloc("__flags__", 4 * 65536)
        self.flags.local.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def alloc(self, name: str, nbytes: int) -> SymmBuffer:
        """Collective: every rank of the group must call it with the same name and size, in the same order."""
        import torch.distributed._symmetric_memory as symm_mem

        buf = self._buffers.get(name)
        if buf is not None and buf.local.numel() >= nbytes:
            return buf
        nbytes = (nbytes + 4095) // 4096 * 4096
        guarded = debug.enabled()
        total = nbytes + (2 * debug.GUARD_BYTES if guarded else 0)
        try:  # older torch versions want the group registered first; newer ones ignore / deprecate the call
            import warnings

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        t = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        handle = symm_mem.rendezvous(t, self.group)
        buf = SymmBuffer(t, handle, self.world, nbytes, debug.Canary(t, nbytes) if guarded else None)
        self._buffers[name] = buf
        return buf

    def verify_guards(self) -> None:
        """Debug mode: raise if anything (this rank or a peer) wrote outside one of this group's buffers."""
        torch.cuda.synchronize(self.device)
        for name, buf in self._buffers.items():
            if buf.guard is not None:
                buf.guard.verify(name)

    def get(self, name: str) -> Optional[SymmBuffer]:
        return self._buffers.get(name)


def group_for(topo: ParallelTopology, axis: str) -> SymmGroup:
    if axis == "ddp" and topo.ep_from_dp:
        axis = "dp"  # the same ranks and the same communicator: one set of flag words
    ranks = tuple(topo.axis_ranks(axis))
    key = (axis, ranks)
    g = _GROUPS.get(key)
    if g is None:
        g = SymmGroup(_axis_group(topo, axis), ranks, topo.device)
        _GROUPS[key] = g
    return g


def disable(reason: str) -> None:
    """Turn the peer-memory paths off for the rest of the process (e.g. after a rendezvous failure)."""
    global _DISABLED_REASON
    _DISABLED_REASON = reason
