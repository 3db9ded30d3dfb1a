"""The allocation-free row-plan entry point, called through its exported C symbol.

Some users of this library cannot allocate GPU memory at call time: a plugin inside another runtime with a
fixed budget, a latency-critical loop that must stay off the allocator lock, a host that already owns the whole
GPU.  For them ``cmoe_moe_plan_noalloc`` keeps its temporary histogram in a fixed array inside the library.  This
test checks that it writes exactly what the regular entry point writes, twice in a row (the array is shared and
keeps the previous call's contents), and that it refuses a problem that does not fit the array.

The file name sorts last so that a run that stops at the first failure has already run everything else.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

CMOE_NOALLOC_OK, CMOE_NOALLOC_BAD_ARGUMENT, CMOE_NOALLOC_TOO_LARGE = 0, 1, 2


def _lib():
    from composed_mixture_of_experts_engine_b200.ops import _ext

    _ext.ext()  # builds if needed and loads the extension (and libtorch) into the process
    lib = ctypes.CDLL(str(_ext._so_path()))
    fn = lib.cmoe_moe_plan_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_longlong] + [ctypes.c_void_p] * 7 + \
                  [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    lib.cmoe_moe_plan_noalloc_words.restype = ctypes.c_size_t
    lib.cmoe_moe_plan_noalloc_words.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return lib


def _outputs(n_slots, n_local, cap_rows):
    i32 = dict(device="cuda", dtype=torch.int32)
    return dict(slot_row=torch.full((n_slots,), -7, **i32), row_slot=torch.full((cap_rows,), -7, **i32),
                group_offsets=torch.full((n_local + 1,), -7, **i32), tile_group=torch.full((cap_rows // 128,), -7, **i32),
                num_m_tiles=torch.full((1,), -7, **i32), counts_kept=torch.full((n_local,), -7, **i32))


@pytest.mark.parametrize("N,K,E,cap", [(3000, 2, 16, 0), (2048, 8, 64, 0), (1500, 2, 8, 90)])
def test_noalloc_plan_matches_regular_entry_point(N, K, E, cap):
    from composed_mixture_of_experts_engine_b200.ops import _ext

    ext, lib = _ext.ext(), _lib()
    per_k = 1 if cap > 0 else 0
    cap_rows = (N * K + E * 127 + 127) // 128 * 128
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):  # two calls in a row: the second one meets the first one's leftovers in the array
        torch.manual_seed(100 * call + N)
        idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(N)]).to(torch.int32).contiguous()
        want = _outputs(N * K, E, cap_rows)
        scratch = torch.empty(ext.moe_plan_scratch_words(N * K, E, K, bool(per_k)), device="cuda", dtype=torch.int32)
        ext.moe_plan(idx, K, E, 0, E, bool(per_k), cap, want["slot_row"], want["row_slot"], want["group_offsets"],
                     want["tile_group"], want["num_m_tiles"], want["counts_kept"], scratch, None)
        got = _outputs(N * K, E, cap_rows)
        dropped = torch.zeros(1, device="cuda", dtype=torch.int32)
        err = ctypes.c_int(0)
        rc = lib.cmoe_moe_plan_noalloc(idx.data_ptr(), N * K, K, E, 0, E, per_k, cap, cap_rows,
                                       got["slot_row"].data_ptr(), got["row_slot"].data_ptr(),
                                       got["group_offsets"].data_ptr(), got["tile_group"].data_ptr(),
                                       got["num_m_tiles"].data_ptr(), got["counts_kept"].data_ptr(),
                                       dropped.data_ptr(), stream, ctypes.byref(err))
        assert rc == CMOE_NOALLOC_OK and err.value == 0
        torch.cuda.synchronize()
        assert int(dropped) == 0  # the row buffer was sized for the worst case
        for name in want:
            assert torch.equal(got[name], want[name]), f"call {call}: {name} differs"
        assert int(got["num_m_tiles"]) > 0


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib = _lib()
    n_slots, n_local, K = 1 << 24, 256, 8  # far beyond the fixed array
    assert lib.cmoe_moe_plan_noalloc_words(n_slots, n_local, K, 1) > (1 << 20)
    t = torch.zeros(1024, device="cuda", dtype=torch.int32)
    p = t.data_ptr()
    err = ctypes.c_int(0)
    rc = lib.cmoe_moe_plan_noalloc(p, n_slots, K, n_local, 0, n_local, 1, 4, 128 * 1024, p, p, p, p, p, p, None, None,
                                   ctypes.byref(err))
    assert rc == CMOE_NOALLOC_TOO_LARGE
    rc = lib.cmoe_moe_plan_noalloc(None, 16, 2, 4, 0, 4, 0, 0, 128, p, p, p, p, p, p, None, None, ctypes.byref(err))
    assert rc == CMOE_NOALLOC_BAD_ARGUMENT
    # experts [3, 3 + 4) do not lie inside [0, 4); a negative capacity makes no sense either
    rc = lib.cmoe_moe_plan_noalloc(p, 16, 2, 4, 3, 4, 0, 0, 128, p, p, p, p, p, p, None, None, ctypes.byref(err))
    assert rc == CMOE_NOALLOC_BAD_ARGUMENT
    rc = lib.cmoe_moe_plan_noalloc(p, 16, 2, 4, 0, 4, 1, -1, 128, p, p, p, p, p, p, None, None, ctypes.byref(err))
    assert rc == CMOE_NOALLOC_BAD_ARGUMENT
    torch.cuda.synchronize()
    assert int(t.abs().sum()) == 0  # nothing was launched
