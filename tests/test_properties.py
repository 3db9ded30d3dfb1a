"""Property-based invariants (Hypothesis, 50 examples each): conservation, normalisation, index range, finiteness over
input scales, complete and balanced expert ownership, config validity (reference: tests/test_properties.py)."""


import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from composed_mixture_of_experts_engine_b200.ops.moe_router import moe_topk_route
from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, ParallelTopology
from composed_mixture_of_experts_engine_b200.parallel.moe_layer import compute_capacity_drop_mask
from composed_mixture_of_experts_engine_b200.utils.config import ConfigValidationError, MoEConfig

pytestmark = pytest.mark.cpu
FAST = settings(max_examples=50, deadline=None)


@FAST
@given(n=st.integers(1, 96), h=st.sampled_from([8, 16, 40]), e=st.integers(1, 24), seed=st.integers(0, 10**6),
       scale=st.sampled_from([0.01, 0.1, 1.0, 10.0]), data=st.data())
def test_router_invariants(n, h, e, seed, scale, data):
    k = data.draw(st.integers(1, e))
    torch.manual_seed(seed)
    x, w = torch.randn(n, h) * scale, torch.randn(h, e) * scale
    idx, wt = moe_topk_route(x, w, k)
    assert idx.shape == (n, k) and int(idx.min()) >= 0 and int(idx.max()) < e
    assert int(torch.bincount(idx.flatten(), minlength=e).sum()) == n * k
    assert torch.isfinite(wt).all() and torch.allclose(wt.sum(-1), torch.ones(n), atol=1e-4)
    assert all(len(set(r)) == k for r in idx.tolist())
    assert bool((wt[:, :-1] >= wt[:, 1:] - 1e-6).all())  # descending gate weights


@FAST
@given(total=st.integers(1, 300), ep=st.integers(1, 16))
def test_expert_ownership_complete_and_balanced(total, ep):
    owned = [ParallelTopology(ep, r, 1, ep).experts_on_this_rank(total) for r in range(ep)]
    assert sorted(sum(owned, [])) == list(range(total))
    sizes = [len(o) for o in owned]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


@FAST
@given(n=st.integers(1, 64), k=st.integers(1, 4), e=st.integers(4, 12), cap=st.integers(0, 20), seed=st.integers(0, 999))
def test_capacity_mask_never_keeps_more_than_capacity(n, k, e, cap, seed):
    torch.manual_seed(seed)
    idx = torch.randint(0, e, (n, k))
    keep = ~compute_capacity_drop_mask(idx, e, cap)
    for col in range(k):
        kept = torch.bincount(idx[:, col][keep[:, col]], minlength=e)
        assert int(kept.max()) <= cap
        total = torch.bincount(idx[:, col], minlength=e)
        assert torch.equal(kept, torch.clamp(total, max=cap))  # first come first served keeps exactly min(count, cap)


@settings(max_examples=20, deadline=None)
@given(seed=st.integers(0, 999), scale=st.sampled_from([0.01, 1.0, 10.0]))
def test_layer_output_is_finite(seed, scale):
    torch.manual_seed(seed)
    layer = DistributedMoELayer(16, 32, 4, 2)
    y = layer(torch.randn(3, 5, 16) * scale)
    assert torch.isfinite(y).all()


@FAST
@given(h=st.integers(1, 64), e=st.integers(1, 32), k=st.integers(1, 40))
def test_config_validity_matches_rules(h, e, k):
    ok = (k <= e) and ((h * 8) % 8 == 0)
    try:
        MoEConfig.from_dict({"model": dict(hidden_dim=h * 8, num_experts=e, top_k=k, num_heads=1)})
        assert ok
    except ConfigValidationError:
        assert not ok


def test_expert_parallel_buffer_sizing(monkeypatch):
    """Row capacity of the expert-parallel buffers: a multiple of the 128-row tile, at least the expected rows plus one
    tile of padding per local expert, never above the worst case (every slot routed here), scaled by the factor."""
    from composed_mixture_of_experts_engine_b200.ops.kernels import ep_buffer_rows, plan_capacity_rows

    monkeypatch.delenv("CMOE_EP_BUFFER_FACTOR", raising=False)
    for n_slots, n_local in ((1, 1), (1000, 8), (131072, 16), (7, 64)):
        cap = plan_capacity_rows(n_slots, n_local)
        assert cap % 128 == 0 and cap >= n_slots + n_local * 127 and cap - (n_slots + n_local * 127) < 128
    expected, n_local, worst = 131072, 8, 8 * 131072
    rows = ep_buffer_rows(expected, n_local, worst)
    assert rows % 128 == 0 and rows >= int(1.5 * expected) + n_local * 128 and rows < worst
    assert ep_buffer_rows(expected, n_local, expected) == plan_capacity_rows(expected, n_local)  # capped by the worst case
    monkeypatch.setenv("CMOE_EP_BUFFER_FACTOR", "1.0")
    assert ep_buffer_rows(expected, n_local, worst) < rows
