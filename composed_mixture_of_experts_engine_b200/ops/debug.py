"""Debug-time index and memory checks (``CMOE_DEBUG_BOUNDS=1``).

The reference has no sanitizer mode of any kind; its safety nets are run-time asserts on routing results
(pkg/kernels/moe_router.py:693-700, pkg/distributed/moe_layer.py:355-358).  The kernels here take row indices that
other kernels computed (the row plan) and write into memory that other GPUs map, so a debug mode checks both before
anything can go wrong on the device:

* ``check_plan``: every index of a row plan is validated with ordinary tensor ops before a gather / GEMM / combine
  kernel consumes it (slot -> row and row -> slot tables in range and inverse to each other, tile table consistent
  with the expert offsets, live tiles within the buffer).  The first violation raises ``PlanBoundsError`` naming the
  table, the position and the value: the bad index never reaches a kernel.
* ``Canary``: guard bands around a buffer (used for the symmetric buffers that peers write into); ``verify`` reports
  the first guard byte that changed, i.e. a write that left its buffer.

Both cost a host synchronisation per call and are meant for tests and bring-up on small shapes, never for timing.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

GUARD_BYTES = 4096
GUARD_PATTERN = 0xA5


def enabled() -> bool:
    return os.environ.get("CMOE_DEBUG_BOUNDS", "0") not in ("", "0")


class PlanBoundsError(RuntimeError):
    """A row plan holds an index outside its table (the message names table, position and value)."""


class GuardBandError(RuntimeError):
    """Bytes outside a guarded buffer were overwritten."""


def _first_bad(mask: torch.Tensor) -> Optional[int]:
    bad = torch.nonzero(mask.reshape(-1), as_tuple=False)
    return int(bad[0]) if bad.numel() else None


def check_plan(slot_row: torch.Tensor, row_slot: torch.Tensor, tile_group: torch.Tensor, num_m_tiles: torch.Tensor,
               group_offsets: torch.Tensor, n_local: int, cap_rows: int, n_slots: Optional[int] = None) -> None:
    """Validate one row plan.  ``slot_row`` [n_slots] (row of each (token, k) slot or -1), ``row_slot`` [cap_rows]
    (slot of each row or -1), ``tile_group`` [cap_rows / 128] (expert of each 128-row tile or -1), ``num_m_tiles``
    [1], ``group_offsets`` [n_local + 1]."""
    n_slots = int(slot_row.numel()) if n_slots is None else n_slots
    tiles = int(num_m_tiles.reshape(-1)[0])
    if tiles < 0 or tiles * 128 > cap_rows or tiles > tile_group.numel():
        raise PlanBoundsError(f"num_m_tiles = {tiles} does not fit a buffer of {cap_rows} rows")
    sr = slot_row.reshape(-1)[:n_slots].long()
    i = _first_bad((sr < -1) | (sr >= tiles * 128))
    if i is not None:
        raise PlanBoundsError(f"slot_row[{i}] = {int(sr[i])} is outside [-1, {tiles * 128})")
    rs = row_slot.reshape(-1)[: tiles * 128].long()
    i = _first_bad((rs < -1) | (rs >= n_slots))
    if i is not None:
        raise PlanBoundsError(f"row_slot[{i}] = {int(rs[i])} is outside [-1, {n_slots})")
    # the two tables are inverse to each other wherever both are set
    live = torch.nonzero(sr >= 0, as_tuple=False).reshape(-1)
    if live.numel():
        back = rs[sr[live]]
        i = _first_bad(back != live)
        if i is not None:
            s = int(live[i])
            raise PlanBoundsError(f"slot {s} maps to row {int(sr[s])}, but that row maps back to slot {int(back[i])}")
    tg = tile_group.reshape(-1)[:tiles].long()
    i = _first_bad((tg < -1) | (tg >= n_local))
    if i is not None:
        raise PlanBoundsError(f"tile_group[{i}] = {int(tg[i])} is outside [-1, {n_local})")
    go = group_offsets.reshape(-1).long()
    if go.numel() != n_local + 1 or int(go[0]) != 0:
        raise PlanBoundsError(f"group_offsets has {go.numel()} entries starting at {int(go[0]) if go.numel() else None}")
    i = _first_bad((go[1:] < go[:-1]) | (go % 128 != 0)[1:] | (go[1:] > cap_rows))
    if i is not None:
        raise PlanBoundsError(f"group_offsets[{i + 1}] = {int(go[i + 1])} (previous {int(go[i])}, buffer {cap_rows})")
    if int(go[-1]) != tiles * 128:
        raise PlanBoundsError(f"group_offsets end at {int(go[-1])} but {tiles} tiles are live")
    # every live tile lies inside the segment of the expert it names
    if tiles:
        t0 = torch.arange(tiles, device=tg.device) * 128
        named = tg.clamp(min=0)
        inside = (t0 >= go[named]) & (t0 < go[named + 1])
        i = _first_bad((tg >= 0) & ~inside)
        if i is not None:
            raise PlanBoundsError(f"tile {i} names expert {int(tg[i])} whose rows are [{int(go[tg[i]])}, "
                                  f"{int(go[tg[i] + 1])})")


class Canary:
    """Guard bands of ``GUARD_BYTES`` before and after the useful part of a byte buffer."""

    def __init__(self, full: torch.Tensor, nbytes: int):
        if full.dtype != torch.uint8 or full.numel() < nbytes + 2 * GUARD_BYTES:
            raise ValueError("guarded buffers are uint8 tensors with room for both guard bands")
        self.full, self.nbytes = full, nbytes
        self.front = full[:GUARD_BYTES]
        self.back = full[GUARD_BYTES + nbytes: GUARD_BYTES + nbytes + GUARD_BYTES]
        self.front.fill_(GUARD_PATTERN)
        self.back.fill_(GUARD_PATTERN)

    @property
    def inner(self) -> torch.Tensor:
        return self.full[GUARD_BYTES: GUARD_BYTES + self.nbytes]

    def verify(self, name: str = "buffer") -> None:
        for label, band, base in (("before", self.front, -GUARD_BYTES), ("after", self.back, self.nbytes)):
            i = _first_bad(band != GUARD_PATTERN)
            if i is not None:
                raise GuardBandError(f"{name}: byte at offset {base + i} ({label} the buffer) was overwritten "
                                     f"with {int(band[i])}")
