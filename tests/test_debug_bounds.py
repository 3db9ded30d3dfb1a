"""The debug-mode index checks of the row plan and the guard bands around buffers (CPU tensors; the same code runs on
device tensors when ``CMOE_DEBUG_BOUNDS=1``)."""

from __future__ import annotations

import pytest
import torch

from composed_mixture_of_experts_engine_b200.ops import debug


def _plan(idx: torch.Tensor, n_experts: int):
    """Expert-sorted, 128-row-padded plan of ``idx`` [N, K] built with plain tensor ops."""
    N, K = idx.shape
    flat = idx.reshape(-1)
    counts = torch.bincount(flat, minlength=n_experts)
    padded = (counts + 127) // 128 * 128
    offs = torch.zeros(n_experts + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(padded, 0)
    cap = int(offs[-1]) + 256
    slot_row = torch.empty(N * K, dtype=torch.int32)
    row_slot = torch.full((cap,), -1, dtype=torch.int32)
    fill = offs[:-1].clone().long()
    for s, e in enumerate(flat.tolist()):
        slot_row[s] = fill[e]
        row_slot[fill[e]] = s
        fill[e] += 1
    tiles = int(offs[-1]) // 128
    tile_group = torch.full((cap // 128,), -1, dtype=torch.int32)
    for e in range(n_experts):
        tile_group[int(offs[e]) // 128: int(offs[e + 1]) // 128] = e
    return dict(slot_row=slot_row, row_slot=row_slot, tile_group=tile_group,
                num_m_tiles=torch.tensor([tiles], dtype=torch.int32), group_offsets=offs, n_local=n_experts,
                cap_rows=cap)


def test_a_valid_plan_passes_and_each_corruption_is_named():
    torch.manual_seed(0)
    idx = torch.stack([torch.randperm(8)[:2] for _ in range(300)])
    good = _plan(idx, 8)
    debug.check_plan(**good)

    def broken(**change):
        p = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in good.items()}
        for k, (pos, val) in change.items():
            p[k][pos] = val
        return p

    with pytest.raises(debug.PlanBoundsError, match=r"slot_row\[17\] = 999999"):
        debug.check_plan(**broken(slot_row=(17, 999999)))
    with pytest.raises(debug.PlanBoundsError, match=r"row_slot\[3\] = 600"):
        debug.check_plan(**broken(row_slot=(3, 600)))
    with pytest.raises(debug.PlanBoundsError, match="maps back to slot"):
        debug.check_plan(**broken(row_slot=(int(good["slot_row"][5]), 6)))
    with pytest.raises(debug.PlanBoundsError, match=r"tile_group\[0\] = 8"):
        debug.check_plan(**broken(tile_group=(0, 8)))
    with pytest.raises(debug.PlanBoundsError, match="tile 0 names expert 3"):
        debug.check_plan(**broken(tile_group=(0, 3)))
    with pytest.raises(debug.PlanBoundsError, match="num_m_tiles"):
        debug.check_plan(**broken(num_m_tiles=(0, 10_000)))
    with pytest.raises(debug.PlanBoundsError, match="group_offsets"):
        debug.check_plan(**broken(group_offsets=(2, 100)))


def test_guard_bands_report_the_first_stray_byte():
    full = torch.zeros(1000 + 2 * debug.GUARD_BYTES, dtype=torch.uint8)
    c = debug.Canary(full, 1000)
    c.inner.fill_(7)  # writes inside the buffer are fine
    c.verify("x")
    full[debug.GUARD_BYTES + 1000 + 12] = 1  # thirteen bytes past the end
    with pytest.raises(debug.GuardBandError, match="offset 1012"):
        c.verify("x")
    full[debug.GUARD_BYTES + 1000 + 12] = debug.GUARD_PATTERN
    full[debug.GUARD_BYTES - 1] = 0  # one byte before the start
    with pytest.raises(debug.GuardBandError, match="offset -1"):
        c.verify("x")


def test_switch_follows_the_environment(monkeypatch):
    monkeypatch.delenv("CMOE_DEBUG_BOUNDS", raising=False)
    assert not debug.enabled()
    monkeypatch.setenv("CMOE_DEBUG_BOUNDS", "1")
    assert debug.enabled()
