"""Expert-parallel dispatch / combine over the library all-to-all (NCCL on GPUs, gloo on CPU).

Same entry points as the reference (pkg/distributed/expert_parallel.py:70-219):

    received, recv_counts, event, ms = all_to_all_dispatch(tokens_sorted, send_counts, topology)
    combined, ms                     = all_to_all_combine(expert_out, recv_counts, send_counts, topology, event)

with two differences: both are differentiable (the backward of a dispatch is the reversed exchange), and
neither waits for the GPU on the host (the reference synchronised on a CUDA event after every exchange,
``expert_parallel.py:128,207``; here ``ms`` is 0.0 unless ``timed=True`` is asked for).  Identity at ep == 1.

This module is the baseline path: the CPU/gloo runs, the multi-rank oracle in the tests and the comparator
for the fused peer-memory kernels (``symm_ep``) that ``DistributedMoELayer`` uses on NVLink-connected GPUs.
"""

from __future__ import annotations

from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from . import collectives as C
from .mesh import ParallelTopology, ep_process_group

__all__ = ["all_to_all_dispatch", "all_to_all_combine", "_CommStream"]

Counts = Union[torch.Tensor, List[int]]


class _CommStream:
    """One high-priority side stream per device for library collectives that should overlap compute."""

    _streams = {}

    @classmethod
    def get(cls, device: torch.device):
        if device.type != "cuda":
            return None
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._streams:
            cls._streams[idx] = torch.cuda.Stream(device=idx, priority=-1)
        return cls._streams[idx]


def _as_list(counts: Counts) -> List[int]:
    return [int(c) for c in (counts.tolist() if isinstance(counts, torch.Tensor) else counts)]


def _inactive(topology: Optional[ParallelTopology]) -> bool:
    return topology is None or topology.ep_size == 1 or not dist.is_initialized()


def all_to_all_dispatch(tokens_sorted: torch.Tensor, send_counts: Counts, topology: Optional[ParallelTopology],
                        recv_counts: Optional[Counts] = None, timed: bool = False
                        ) -> Tuple[torch.Tensor, torch.Tensor, Optional[object], float]:
    """Send ``send_counts[r]`` consecutive rows of ``tokens_sorted`` to EP rank r.

    Returns the received rows (grouped by source rank), the per-source row counts, a CUDA event recorded after
    the exchange (``None`` on CPU) and the elapsed milliseconds (only measured when ``timed``).
    """
    if _inactive(topology):
        cnt = send_counts if isinstance(send_counts, torch.Tensor) else torch.tensor(send_counts, dtype=torch.int64)
        return tokens_sorted, cnt, None, 0.0
    group = ep_process_group(topology)
    send = _as_list(send_counts)
    if sum(send) != tokens_sorted.shape[0]:
        raise ValueError(f"send_counts sum to {sum(send)} but {tokens_sorted.shape[0]} rows were given")
    if recv_counts is None:
        sc = torch.tensor(send, dtype=torch.int64, device=tokens_sorted.device)
        recv = _as_list(C.exchange_counts(sc, group))
    else:
        recv = _as_list(recv_counts)
    ev0 = ev1 = None
    if timed and tokens_sorted.is_cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    received = C.all_to_all_rows(tokens_sorted, send, recv, group)
    event, ms = None, 0.0
    if tokens_sorted.is_cuda:
        event = ev1 if ev1 is not None else torch.cuda.Event()
        event.record()
        if timed:
            event.synchronize()
            ms = ev0.elapsed_time(event)
    return received, torch.tensor(recv, dtype=torch.int64), event, ms


def all_to_all_combine(expert_out: torch.Tensor, recv_counts: Counts, send_counts: Counts,
                       topology: Optional[ParallelTopology], wait_event: Optional[object] = None,
                       timed: bool = False) -> Tuple[torch.Tensor, float]:
    """Inverse of :func:`all_to_all_dispatch`: rows go back to the ranks they came from, in their original order."""
    if _inactive(topology):
        return expert_out, 0.0
    group = ep_process_group(topology)
    if wait_event is not None and expert_out.is_cuda:
        torch.cuda.current_stream().wait_event(wait_event)
    ev0 = ev1 = None
    if timed and expert_out.is_cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    combined = C.all_to_all_rows(expert_out, _as_list(recv_counts), _as_list(send_counts), group)
    ms = 0.0
    if ev1 is not None:
        ev1.record()
        ev1.synchronize()
        ms = ev0.elapsed_time(ev1)
    return combined, ms
