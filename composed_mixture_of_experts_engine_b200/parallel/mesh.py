"""Rank topology of the 4-D mesh (data x tensor x pipeline x expert) and its process groups.

Keeps the reference's ``ParallelTopology`` / ``build_topology`` / ``tp_process_group`` /
``pp_process_group`` surface and rank-coordinate formulas (``pkg/distributed/mesh.py:60-326``):
``dp = (r // (tp*pp*ep)) % dp``, ``tp = (r // (pp*ep)) % tp``, ``pp = (r // ep) % pp``, ``ep = r % ep``,
contiguous expert ownership with the remainder on the lowest EP ranks, and the degenerate one-rank
topology whenever the world size is 1.

Differences, all opt-in or fixes:

* ``ep_from_dp=True``: the expert-parallel group is carved out of the data-parallel axis
  (world = dp * tp * pp, ``ep_rank = dp_rank % ep``), which is what a dp=8 x ep=8 job on 8 GPUs means.
* Every axis gets an explicit process group (``AxisGroups``) created by all ranks in the same order;
  the reference's hand-built TP rank list ignored the pipeline axis (``mesh.py:188-198``).
* ``torch.cuda.set_device`` is called for CUDA topologies (the reference never did, ``mesh.py:315-316``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = [
    "ParallelTopology",
    "AxisGroups",
    "build_topology",
    "tp_process_group",
    "pp_process_group",
    "ep_process_group",
    "dp_process_group",
    "edp_process_group",
    "ddp_process_group",
    "etp_process_group",
]

_TP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}
_PP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


class _AxisHandle:
    def __init__(self, group, ranks: List[int]):
        self._group, self.ranks = group, ranks

    def get_group(self):
        return self._group


class AxisGroups:
    """Process groups of one rank, one per mesh axis, addressable like a DeviceMesh (``mesh["tp"].get_group()``)."""

    def __init__(self) -> None:
        self._axes: Dict[str, _AxisHandle] = {}

    def add(self, axis: str, group, ranks: List[int]) -> None:
        self._axes[axis] = _AxisHandle(group, ranks)

    def __getitem__(self, axis: str) -> _AxisHandle:
        return self._axes[axis]

    def __contains__(self, axis: str) -> bool:
        return axis in self._axes

    def get_group(self, axis: str):
        return self._axes[axis].get_group()

    def ranks(self, axis: str) -> List[int]:
        return self._axes[axis].ranks


@dataclass(frozen=True)
class ParallelTopology:
    """Immutable description of this rank's place in the mesh."""

    world_size: int
    rank: int
    dp_size: int
    ep_size: int
    tp_size: int = 1
    pp_size: int = 1
    mesh: Optional[object] = field(default=None, compare=False, repr=False)
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    ep_from_dp: bool = False

    # ---- coordinates --------------------------------------------------------------------------
    @property
    def _ep_axis(self) -> int:
        return 1 if self.ep_from_dp else self.ep_size

    @property
    def dp_rank(self) -> int:
        return (self.rank // (self.tp_size * self.pp_size * self._ep_axis)) % self.dp_size

    @property
    def tp_rank(self) -> int:
        return (self.rank // (self.pp_size * self._ep_axis)) % self.tp_size

    @property
    def pp_rank(self) -> int:
        return (self.rank // self._ep_axis) % self.pp_size

    @property
    def ep_rank(self) -> int:
        if self.ep_from_dp:
            return self.dp_rank % self.ep_size
        return self.rank % self.ep_size

    def rank_of(self, dp: int, tp: int, pp: int, ep: int = 0) -> int:
        """Global rank at the given coordinates (``ep`` ignored when EP is carved from DP)."""
        a = self._ep_axis
        return ((dp * self.tp_size + tp) * self.pp_size + pp) * a + (0 if self.ep_from_dp else ep)

    def axis_ranks(self, axis: str) -> List[int]:
        """Global ranks of this rank's group along ``axis`` (dp | tp | pp | ep), in axis order."""
        dp, tp, pp, ep = self.dp_rank, self.tp_rank, self.pp_rank, self.ep_rank
        if axis == "dp":
            return [self.rank_of(d, tp, pp, ep) for d in range(self.dp_size)]
        if axis == "tp":
            return [self.rank_of(dp, t, pp, ep) for t in range(self.tp_size)]
        if axis == "pp":
            return [self.rank_of(dp, tp, p, ep) for p in range(self.pp_size)]
        if axis == "ep":
            if self.ep_from_dp:
                base = (dp // self.ep_size) * self.ep_size
                return [self.rank_of(base + e, tp, pp) for e in range(self.ep_size)]
            return [self.rank_of(dp, tp, pp, e) for e in range(self.ep_size)]
        if axis == "edp":  # ranks that hold the same experts (expert-data-parallel replicas)
            if self.ep_from_dp:
                return [self.rank_of(d, tp, pp) for d in range(self.dp_size) if d % self.ep_size == ep]
            return [self.rank_of(d, tp, pp, ep) for d in range(self.dp_size)]
        if axis == "etp":  # expert-parallel x tensor-parallel block: ep-major, tp-minor (index = ep_rank * tp + tp_rank)
            if self.ep_from_dp:
                base = (dp // self.ep_size) * self.ep_size
                return [self.rank_of(base + e, t, pp) for e in range(self.ep_size) for t in range(self.tp_size)]
            return [self.rank_of(dp, t, pp, e) for e in range(self.ep_size) for t in range(self.tp_size)]
        if axis == "ddp":  # ranks that hold the same dense parameters and see different data
            if self.ep_from_dp:
                return self.axis_ranks("dp")
            return [self.rank_of(d, tp, pp, e) for d in range(self.dp_size) for e in range(self.ep_size)]
        raise KeyError(axis)

    def axis_size(self, axis: str) -> int:
        if axis in ("dp", "tp", "pp", "ep"):
            return {"dp": self.dp_size, "tp": self.tp_size, "pp": self.pp_size, "ep": self.ep_size}[axis]
        return len(self.axis_ranks(axis))

    @property
    def data_replicas(self) -> int:
        """How many ranks draw different data for the same dense parameters: ``dp`` when the expert-parallel group
        is carved out of the data-parallel axis, ``dp * ep`` when it is an axis of its own (every expert-parallel
        rank feeds its own tokens into the exchange)."""
        return self.dp_size if self.ep_from_dp else self.dp_size * self.ep_size

    @property
    def data_rank(self) -> int:
        """This rank's index among the ``data_replicas`` (what a data loader seeds or shards by)."""
        return self.axis_ranks("ddp").index(self.rank)

    # ---- expert ownership ---------------------------------------------------------------------
    def experts_on_rank(self, total_experts: int, ep_rank: int) -> List[int]:
        per, rem = divmod(total_experts, self.ep_size)
        start = ep_rank * per + min(ep_rank, rem)
        return list(range(start, start + per + (1 if ep_rank < rem else 0)))

    def experts_on_this_rank(self, total_experts: int) -> List[int]:
        return self.experts_on_rank(total_experts, self.ep_rank)

    # ---- convenience --------------------------------------------------------------------------
    def is_first_pp_stage(self) -> bool:
        return self.pp_rank == 0

    def is_last_pp_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @property
    def expected_world_size(self) -> int:
        base = self.dp_size * self.tp_size * self.pp_size
        return base if self.ep_from_dp else base * self.ep_size

    def validate_world_size(self) -> None:
        if self.expected_world_size != self.world_size:
            how = "dp x tp x pp (ep carved from dp)" if self.ep_from_dp else "dp x ep x tp x pp"
            raise ValueError(
                f"Parallelism product dp({self.dp_size}) × ep({self.ep_size}) × tp({self.tp_size}) × "
                f"pp({self.pp_size}) [{how}] = {self.expected_world_size} != world_size({self.world_size}).\n"
                "Adjust the parallelism config so the product matches the number of GPUs."
            )


def _axis_group(topology: ParallelTopology, axis: str, cache: Dict[Tuple[int, ...], "dist.ProcessGroup"]):
    size = topology.axis_size(axis)
    if size == 1 or not dist.is_initialized():
        return None
    if topology.mesh is not None and axis in topology.mesh:  # type: ignore[operator]
        return topology.mesh[axis].get_group()  # type: ignore[index]
    ranks = tuple(topology.axis_ranks(axis))
    if ranks not in cache:
        cache[ranks] = dist.new_group(ranks=list(ranks))
    return cache[ranks]


def tp_process_group(topology: ParallelTopology):
    """The tensor-parallel group of this rank (``None`` when tp == 1 or no process group exists)."""
    return _axis_group(topology, "tp", _TP_GROUPS)


def pp_process_group(topology: ParallelTopology):
    return _axis_group(topology, "pp", _PP_GROUPS)


_EP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}
_DP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


def ep_process_group(topology: ParallelTopology):
    return _axis_group(topology, "ep", _EP_GROUPS)


def dp_process_group(topology: ParallelTopology):
    return _axis_group(topology, "dp", _DP_GROUPS)


_EDP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


def edp_process_group(topology: ParallelTopology):
    """Ranks holding replicas of this rank's experts (gradients of expert weights are reduced over these)."""
    return _axis_group(topology, "edp", _EDP_GROUPS)


_DDP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


def ddp_process_group(topology: ParallelTopology):
    """Ranks holding replicas of this rank's dense parameters (their gradients are reduced over these): the
    data-parallel group, times the expert-parallel group when that is an axis of its own."""
    return _axis_group(topology, "ddp", _DDP_GROUPS)


_ETP_GROUPS: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


def etp_process_group(topology: ParallelTopology):
    """The expert-parallel x tensor-parallel block of this rank: the ranks that together hold every (expert, FFN
    slice) pair, over which the MoE layer exchanges token rows when sequence parallelism hands it sequence shards."""
    return _axis_group(topology, "etp", _ETP_GROUPS)


def _build_axis_groups(probe: ParallelTopology) -> AxisGroups:
    """Create every axis group of every rank, in an order that is the same on all ranks."""
    groups = AxisGroups()
    world = probe.world_size
    for axis in ("dp", "tp", "pp", "ep", "edp", "ddp", "etp"):
        if axis == "ddp" and probe.ep_from_dp:  # the same ranks as "dp": share its communicator
            if "dp" in groups:
                groups.add("ddp", groups.get_group("dp"), groups.ranks("dp"))
            continue
        if axis == "etp" and (probe.tp_size == 1 or probe.ep_size == 1):
            # one of the two factors is trivial: the block is the other axis' group
            other = "ep" if probe.tp_size == 1 else "tp"
            if other in groups:
                groups.add("etp", groups.get_group(other), groups.ranks(other))
            continue
        seen = set()
        for r in range(world):
            t = ParallelTopology(world, r, probe.dp_size, probe.ep_size, probe.tp_size, probe.pp_size,
                                 ep_from_dp=probe.ep_from_dp)
            ranks = tuple(t.axis_ranks(axis))
            if ranks in seen:
                continue
            seen.add(ranks)
            g = dist.new_group(ranks=list(ranks)) if len(ranks) > 1 else None
            if probe.rank in ranks:
                groups.add(axis, g, list(ranks))
    return groups


def build_topology(
    dp_size: int,
    ep_size: int,
    tp_size: int = 1,
    pp_size: int = 1,
    device_type: str = "cuda",
    ep_from_dp: bool = False,
) -> ParallelTopology:
    """Describe this rank and build its process groups.

    With a world size of 1 (or no initialised process group) the degenerate topology
    ``dp = ep = tp = pp = 1`` is returned whatever sizes were asked for, so that single-process code
    and tests run unchanged.
    """
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    use_cuda = device_type == "cuda" and torch.cuda.is_available()
    if world == 1:
        dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        return ParallelTopology(1, 0, 1, 1, 1, 1, mesh=None, device=dev)

    probe = ParallelTopology(world, rank, dp_size, ep_size, tp_size, pp_size, ep_from_dp=ep_from_dp)
    if probe.expected_world_size != world:
        how = "dp × tp × pp" if ep_from_dp else "dp × tp × pp × ep"
        raise ValueError(
            f"dp({dp_size}) × tp({tp_size}) × pp({pp_size}) × ep({ep_size}) [{how}] = "
            f"{probe.expected_world_size} must equal world_size({world}).\n"
            "Adjust parallelism config to match the number of available GPUs."
        )
    if ep_from_dp and dp_size % ep_size != 0:
        raise ValueError(f"ep_from_dp needs dp({dp_size}) divisible by ep({ep_size})")
    if use_cuda:
        local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    groups = _build_axis_groups(probe)
    return ParallelTopology(world, rank, dp_size, ep_size, tp_size, pp_size, mesh=groups, device=dev,
                            ep_from_dp=ep_from_dp)
