"""Thin, allocation-aware Python wrappers over the sm_100a extension entry points.

Nothing here is differentiable; the autograd functions live in ``functional.py``.  Every wrapper
launches on the current stream and returns at once.  Waits inside the kernels are bounded; a wait that
ran out sets a status word that :func:`check_status` turns into :class:`KernelTimeoutError`.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _ext

GEMM_DENSE, GEMM_GROUPED_M, GEMM_GROUPED_K = 0, 1, 2
EPI_STORE, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2

STATUS_NAMES = {
    0: "ok",
    1: "timeout: shared-memory stage never filled (TMA)",
    2: "timeout: shared-memory stage never released",
    3: "timeout: accumulator never committed",
    4: "timeout: accumulator never drained",
    5: "timeout: peer flag never written",
    6: "bad argument",
    7: "a row plan or routing table named a rank or row outside the buffers (the access was skipped)",
}


class KernelTimeoutError(RuntimeError):
    """A bounded wait inside a kernel ran out; the CUDA context is still usable."""


_status: Dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The per-device int32 status word that all launches of this package share."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
        _ext.ext().set_peer_status_word(t)  # the peer row kernels record bad indices in the same word
    return t


def check_status(device: Optional[torch.device] = None, reset: bool = True) -> None:
    """Synchronises with the device and raises if any kernel since the last check recorded an error."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    t = status_word(dev)
    code = int(t.item())
    if code != 0:
        if reset:
            t.zero_()
        raise KernelTimeoutError(f"kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


def gemm(
    A: torch.Tensor,
    B: torch.Tensor,
    D: torch.Tensor,
    *,
    mode: int = GEMM_DENSE,
    epilogue: int = EPI_STORE,
    M: int = 0,
    N: int = 0,
    K: int = 0,
    a_mn: bool = False,
    b_mn: bool = False,
    groups: int = 1,
    b_group_rows: int = 0,
    split_n: int = 0,
    tile_group: Optional[torch.Tensor] = None,
    num_m_tiles: Optional[torch.Tensor] = None,
    max_m_tiles: int = 0,
    group_offsets: Optional[torch.Tensor] = None,
    d_group_stride: int = 0,
    accumulate: bool = False,
    aux_in: Optional[torch.Tensor] = None,
    aux_out: Optional[torch.Tensor] = None,
    ready_flags: Optional[torch.Tensor] = None,
    ready_stride: int = 0,
    ready_count: int = 0,
    ready_target: int = 0,
    timeout_ns: int = 0,
) -> torch.Tensor:
    _ext.ext().gemm(
        A, B, D, mode, epilogue, M, N, K, a_mn, b_mn, groups, b_group_rows, split_n, tile_group, num_m_tiles,
        max_m_tiles, group_offsets, d_group_stride, accumulate, aux_in, aux_out, ready_flags, ready_stride,
        ready_count, ready_target, status_word(A.device), timeout_ns,
    )
    return D


def linear_nt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
              out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (the nn.Linear contraction) on the tcgen05 GEMM."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=out_dtype)
    return gemm(x, w, out, M=M, N=N, K=K, accumulate=accumulate)


def linear_nn(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
              out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[K, N] (w read N-major, no transpose copy)."""
    M, K = x.shape
    N = w.shape[1]
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=out_dtype)
    return gemm(x, w, out, M=M, N=N, K=K, b_mn=True, accumulate=accumulate)


_offsets_cache: Dict[Tuple[int, Tuple[int, ...]], torch.Tensor] = {}


def _offsets_i32(device: torch.device, offs: Tuple[int, ...]) -> torch.Tensor:
    """Device copy of a short host list of row offsets, made once per distinct list (a fresh ``torch.tensor``
    per call would be a pageable host-to-device copy in the middle of the backward pass)."""
    key = (device.index or 0, offs)
    t = _offsets_cache.get(key)
    if t is None:
        if len(_offsets_cache) > 256:
            _offsets_cache.clear()
        t = torch.tensor(offs, device=device, dtype=torch.int32)
        _offsets_cache[key] = t
    return t


def linear_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
              splits: int = 0) -> torch.Tensor:
    """out[M, N] (fp32) = a[R, M]^T @ b[R, N]: the weight-gradient contraction over R rows.

    The R rows are cut into ``splits`` chunks (multiples of 64 rows) that run as separate tiles and
    are summed afterwards, so that small outputs still fill the GPU.
    """
    R, M = a.shape
    N = b.shape[1]
    if splits <= 0:
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        splits = max(1, min(R // 512 if R >= 512 else 1, (148 + tiles - 1) // tiles))
    chunk = ((R + splits - 1) // splits + 63) // 64 * 64
    offs = tuple(min(i * chunk, R) for i in range(splits)) + (R,)
    offs_t = _offsets_i32(a.device, offs)
    part = torch.empty(splits, M, N, device=a.device, dtype=torch.float32)
    gemm(a, b, part, mode=GEMM_GROUPED_K, M=M, N=N, a_mn=True, b_mn=True, groups=splits, group_offsets=offs_t,
         d_group_stride=M * N)
    red = part[0] if splits == 1 else part.sum(0)
    if out is None:
        return red
    if accumulate:
        out.add_(red.to(out.dtype))
    else:
        out.copy_(red)
    return out


def linear_tn_acc(a: torch.Tensor, b: torch.Tensor, acc: torch.Tensor, accumulate: bool = True) -> torch.Tensor:
    """acc[M, N] (fp32, in place) += a[R, M]^T @ b[R, N] with the addition done by the kernel's TMA reduce-add
    epilogue (no read-modify-write pass over ``acc`` on the SMs, no temporary); ``accumulate=False`` stores."""
    R, M = a.shape
    N = b.shape[1]
    gemm(a, b, acc, mode=GEMM_GROUPED_K, M=M, N=N, a_mn=True, b_mn=True, groups=1,
         group_offsets=_offsets_i32(a.device, (0, R)), d_group_stride=M * N, accumulate=accumulate)
    return acc


_overflow: Dict[int, torch.Tensor] = {}


def overflow_counter(device: torch.device) -> torch.Tensor:
    """Per-device counter of (token, slot) pairs that a row plan had to drop because its buffer was too small."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _overflow.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _overflow[idx] = t
    return t


def ep_buffer_rows(n_slots_expected: int, n_local: int, worst_case: int) -> int:
    """Row capacity of expert-parallel buffers: the expected rows times ``CMOE_EP_BUFFER_FACTOR`` (default 1.5)
    plus tile padding, never more than the worst case.  Slots beyond it are dropped and counted."""
    import os

    factor = float(os.environ.get("CMOE_EP_BUFFER_FACTOR", "1.5"))
    want = int(n_slots_expected * factor) + n_local * 128
    return min(plan_capacity_rows(worst_case, n_local), (want + 127) // 128 * 128)


class MoEPlan:
    """Device-resident description of one expert-sorted, 128-row-padded row layout."""

    __slots__ = ("n_tokens", "K", "n_local", "cap_rows", "slot_row", "row_slot", "group_offsets", "tile_group",
                 "num_m_tiles", "counts_kept", "max_m_tiles")

    def __init__(self, n_tokens: int, K: int, n_local: int, cap_rows: int, device: torch.device,
                 slot_row: Optional[torch.Tensor] = None):
        self.n_tokens, self.K, self.n_local, self.cap_rows = n_tokens, K, n_local, cap_rows
        i32 = dict(device=device, dtype=torch.int32)
        self.slot_row = slot_row if slot_row is not None else torch.empty(n_tokens * K, **i32)
        self.row_slot = torch.empty(cap_rows, **i32)
        self.group_offsets = torch.empty(n_local + 1, **i32)
        self.tile_group = torch.empty(cap_rows // 128, **i32)
        self.num_m_tiles = torch.empty(1, **i32)
        self.counts_kept = torch.empty(n_local, **i32)
        self.max_m_tiles = cap_rows // 128


def plan_capacity_rows(n_slots: int, n_local: int) -> int:
    """Worst-case rows of the padded layout: every slot kept plus up to 127 padding rows per expert."""
    return (n_slots + n_local * 127 + 127) // 128 * 128


_scratch: Dict[Tuple[int, int], torch.Tensor] = {}


def _scratch_i32(device: torch.device, words: int) -> torch.Tensor:
    key = (device.index or 0, 0)
    t = _scratch.get(key)
    if t is None or t.numel() < words:
        t = torch.empty(max(words, 1 << 16), device=device, dtype=torch.int32)
        _scratch[key] = t
    return t


def moe_plan(topk_idx: torch.Tensor, num_experts: int, expert_lo: int = 0, n_local: Optional[int] = None,
             capacity: int = 0, cap_rows: Optional[int] = None, slot_row_out: Optional[torch.Tensor] = None
             ) -> MoEPlan:
    """Build the row plan for ``topk_idx`` [N, K] (int32).  ``capacity`` > 0 enables per-(expert, k) FCFS dropping."""
    ext = _ext.ext()
    N, K = topk_idx.shape
    n_local = num_experts if n_local is None else n_local
    if cap_rows is None:
        cap_rows = plan_capacity_rows(N * K, n_local)
    plan = MoEPlan(N, K, n_local, cap_rows, topk_idx.device, slot_row=slot_row_out)
    per_k = capacity > 0
    words = ext.moe_plan_scratch_words(N * K, n_local, K, per_k)
    ext.moe_plan(topk_idx, K, num_experts, expert_lo, n_local, per_k, capacity, plan.slot_row, plan.row_slot,
                 plan.group_offsets, plan.tile_group, plan.num_m_tiles, plan.counts_kept,
                 _scratch_i32(topk_idx.device, words), overflow_counter(topk_idx.device))
    from . import debug

    if debug.enabled():  # validate every index before a gather / GEMM / combine kernel consumes the plan
        debug.check_plan(plan.slot_row, plan.row_slot, plan.tile_group, plan.num_m_tiles, plan.group_offsets, n_local,
                         cap_rows, N * K)
    return plan


def gather_rows(src: torch.Tensor, plan: MoEPlan, slot_scale: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(plan.cap_rows, src.shape[1], device=src.device, dtype=torch.bfloat16)
    _ext.ext().gather_rows(src, plan.row_slot, plan.K, slot_scale, out, plan.num_m_tiles)
    return out


def combine_rows(rows: torch.Tensor, plan: MoEPlan, w: Optional[torch.Tensor], out: Optional[torch.Tensor] = None
                 ) -> torch.Tensor:
    if out is None:
        out = torch.empty(plan.n_tokens, rows.shape[1], device=rows.device, dtype=torch.bfloat16)
    _ext.ext().combine_rows(rows, plan.slot_row, w, out, plan.K)
    return out


def combine_bwd_w(rows: torch.Tensor, plan: MoEPlan, dy: torch.Tensor) -> torch.Tensor:
    dw = torch.empty(plan.n_tokens, plan.K, device=rows.device, dtype=torch.float32)
    _ext.ext().combine_bwd_w(rows, plan.slot_row, dy, dw, plan.K)
    return dw


_tile_ready: Dict[int, torch.Tensor] = {}
_pull_epoch: Dict[int, int] = {}


def gemm_pull(A: torch.Tensor, B: torch.Tensor, D: torch.Tensor, plan: MoEPlan, *, epilogue: int, N: int, K: int,
              groups: int, b_group_rows: int, src_ptrs, slots_per_src: int, pull_K: int, ld_src: int,
              b_mn: bool = False, split_n: int = 0, aux_in: Optional[torch.Tensor] = None,
              aux_out: Optional[torch.Tensor] = None, slot_scale: Optional[torch.Tensor] = None,
              stamps: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped GEMM whose A rows (``plan.row_slot`` -> token rows of the ranks in ``src_ptrs``) are brought in by
    extra warps of the same kernel, tile by tile (fused expert-parallel dispatch).  ``A`` is the destination
    buffer of the pulled rows as well as the GEMM operand.  ``stamps`` (int64[4], see :func:`new_pull_stamps`)
    receives the device timestamps of first / last row pulled and first / last MMA."""
    idx = A.device.index or 0
    ready = _tile_ready.get(idx)
    if ready is None or ready.numel() < 4 * plan.max_m_tiles:  # four flags per 128-row tile (csrc/gemm.cuh)
        ready = torch.zeros(max(4 * plan.max_m_tiles, 65536), device=A.device, dtype=torch.int32)
        _tile_ready[idx] = ready
        _pull_epoch[idx] = 0
    _pull_epoch[idx] = (_pull_epoch[idx] + 1) % (1 << 30)
    if _pull_epoch[idx] == 0:  # wrapped: start over with clean flags
        ready.zero_()
        _pull_epoch[idx] = 1
    _ext.ext().gemm_pull(A, B, D, epilogue, N, K, b_mn, groups, b_group_rows, split_n, plan.tile_group,
                         plan.num_m_tiles, plan.max_m_tiles, aux_in, aux_out, plan.row_slot, list(src_ptrs),
                         slots_per_src, pull_K, slot_scale, ld_src, ready, _pull_epoch[idx], status_word(A.device), 0,
                         stamps)
    return D


_I64_MAX = (1 << 63) - 1


def new_pull_stamps(device: torch.device) -> torch.Tensor:
    """A timestamp record for :func:`gemm_pull`: {first pull, last pull, first MMA, last MMA} in nanoseconds of the
    device's global timer, preset so that the kernel's atomic min / max leave the extremes over all CTAs."""
    return torch.tensor([_I64_MAX, 0, _I64_MAX, 0], dtype=torch.int64, device=device)


def pull_overlap_ratio(stamps: torch.Tensor) -> Optional[float]:
    """Fraction of the row transfer's duration during which the tensor cores of the same launch were at work:
    |[first pull, last pull] intersected with [first MMA, last MMA]| / |[first pull, last pull]|.  One device read.
    ``None`` when the launch recorded nothing (no rows pulled)."""
    p0, p1, m0, m1 = (int(v) for v in stamps.tolist())
    if p0 == _I64_MAX or m0 == _I64_MAX or p1 <= p0:
        return None
    return max(0, min(p1, m1) - max(p0, m0)) / float(p1 - p0)


def gemm_scatter(A: torch.Tensor, B: torch.Tensor, *, N: int, K: int, row_slot: torch.Tensor, slots_per_rank: int,
                 out_ptrs, out_ld: int, plan: Optional[MoEPlan] = None, groups: int = 1, b_group_rows: int = 0,
                 b_mn: bool = False, M: int = 0) -> None:
    """GEMM (grouped by ``plan`` or dense with ``M`` rows) whose epilogue stores output row r in the buffer of rank
    ``row_slot[r] // slots_per_rank`` (one of ``out_ptrs``) at row ``row_slot[r] % slots_per_rank``; rows with a
    negative slot are skipped."""
    dummy = A  # D is not written in scatter mode; any bf16 2-D tensor satisfies the binding's checks
    if plan is not None:
        _ext.ext().gemm_scatter(A, B, dummy, GEMM_GROUPED_M, 0, N, K, b_mn, groups, b_group_rows, plan.tile_group,
                                plan.num_m_tiles, plan.max_m_tiles, row_slot, slots_per_rank, list(out_ptrs), out_ld,
                                status_word(A.device), 0)
    else:
        _ext.ext().gemm_scatter(A, B, dummy, GEMM_DENSE, M, N, K, b_mn, 1, 0, None, None, 0, row_slot, slots_per_rank,
                                list(out_ptrs), out_ld, status_word(A.device), 0)
