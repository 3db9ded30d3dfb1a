"""MoE layer, capacity dropping, topology ownership and TP/SP at tp=1 on the CPU path
(reference: tests/test_distributed.py, test_capacity_dropping.py, test_tensor_parallel.py,
test_sequence_parallel_v03.py)."""


import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from composed_mixture_of_experts_engine_b200.ops.functional import capacity_drop_mask_reference, experts_reference
from composed_mixture_of_experts_engine_b200.parallel import (ColumnParallelLinear, DistributedMoELayer,
                                                              ParallelTopology, RowParallelLinear, build_topology,
                                                              gather_from_sequence_parallel,
                                                              scatter_to_sequence_parallel)
from composed_mixture_of_experts_engine_b200.parallel.moe_layer import (_cumcount, _SwiGLUExpert,
                                                                        compute_capacity_drop_mask)

pytestmark = pytest.mark.cpu


def _dense_oracle(layer, x):
    flat = x.reshape(-1, x.shape[-1])
    idx, w, _ = layer.router(flat)
    y = torch.zeros_like(flat)
    f = layer.w13.shape[1] // 2
    for t in range(flat.shape[0]):
        for k in range(layer.top_k):
            e = int(idx[t, k])
            h = F.silu(flat[t] @ layer.w13[e, :f].t()) * (flat[t] @ layer.w13[e, f:].t())
            y[t] += w[t, k] * (h @ layer.w2[e].t())
    return y.reshape(x.shape)


def test_layer_matches_per_token_oracle_and_shapes():
    torch.manual_seed(0)
    layer = DistributedMoELayer(32, 64, 8, 2)
    x = torch.randn(2, 7, 32)
    y = layer(x)
    assert y.shape == x.shape
    assert torch.allclose(y, _dense_oracle(layer, x), atol=1e-5)
    assert layer(x.reshape(14, 32)).shape == (14, 32)
    with pytest.raises(ValueError):
        layer(torch.randn(32))
    with pytest.raises(ValueError):
        layer(torch.randn(3, 16))


def test_layer_gradients_reach_everything():
    torch.manual_seed(1)
    layer = DistributedMoELayer(32, 64, 4, 2)
    x = torch.randn(3, 5, 32, requires_grad=True)
    layer(x).pow(2).sum().backward()
    for t in (x.grad, layer.router.gate_w.grad, layer.w13.grad, layer.w2.grad):
        assert t is not None and torch.isfinite(t).all() and t.abs().sum() > 0
    assert not torch.isnan(layer(x)).any()


def test_experts_module_list_views():
    layer = DistributedMoELayer(16, 32, 4, 2)
    assert len(layer.experts) == 4 and layer.local_expert_ids == [0, 1, 2, 3]
    e0 = layer.experts[0]
    assert isinstance(e0, _SwiGLUExpert)
    assert isinstance(e0.w_gate, ColumnParallelLinear) and isinstance(e0.w_up, ColumnParallelLinear)
    assert isinstance(e0.w_down, RowParallelLinear)
    assert [n for n, _ in layer.named_parameters()] == ["w13", "w2", "router.gate_w"]
    x = torch.randn(3, 16)
    want = (F.silu(x @ layer.w13[0, :32].t()) * (x @ layer.w13[0, 32:].t())) @ layer.w2[0].t()
    assert torch.allclose(e0(x), want, atol=1e-6)
    assert e0.w_gate.weight.data_ptr() == layer.w13[0].data_ptr()  # a live view, not a copy


def test_custom_experts_switch_to_generic_loop():
    torch.manual_seed(2)

    class Doubler(nn.Module):
        def forward(self, x):
            return 2 * x

    layer = DistributedMoELayer(16, 32, 4, 2)
    layer.experts = nn.ModuleList([Doubler() for _ in range(4)])
    x = torch.randn(6, 16)
    assert torch.allclose(layer(x), 2 * x, atol=1e-5)  # gate weights sum to one


def test_standalone_swiglu_expert():
    e = _SwiGLUExpert(16, 32)
    x = torch.randn(4, 16)
    want = F.linear(F.silu(F.linear(x, e.w_gate.weight)) * F.linear(x, e.w_up.weight), e.w_down.weight)
    assert torch.allclose(e(x), want, atol=1e-6)
    by_name = _SwiGLUExpert(hidden_dim=16, ffn_dim=32, topology=None)  # the reference's keyword names
    assert by_name.w_gate.weight.shape == (32, 16) and by_name.w_down.weight.shape == (16, 32)


@pytest.mark.parametrize("ids,want", [([0, 0, 1, 0, 1, 2], [0, 1, 0, 2, 1, 0]), ([5], [0]), ([], []),
                                       ([3, 3, 3], [0, 1, 2])])
def test_cumcount(ids, want):
    assert _cumcount(torch.tensor(ids, dtype=torch.long)).tolist() == want


def test_capacity_mask_per_k_column():
    idx = torch.tensor([[0, 1], [0, 1], [0, 0], [1, 0]])
    m = compute_capacity_drop_mask(idx, 2, 2)
    # column 0: expert 0 seen at rows 0,1,2 -> row 2 dropped; column 1: expert 1 rows 0,1; expert 0 rows 2,3
    assert m.tolist() == [[False, False], [False, False], [True, False], [False, False]]
    assert torch.equal(m, capacity_drop_mask_reference(idx, 2, 2))
    assert compute_capacity_drop_mask(idx, 2, 0).all()
    with pytest.raises(ValueError):
        compute_capacity_drop_mask(idx[0], 2, 1)


def test_layer_capacity_dropping_deterministic():
    torch.manual_seed(3)
    layer = DistributedMoELayer(16, 32, 4, 2, capacity_factor=0.5, capacity_dropping=True)
    x = torch.randn(64, 16)
    y1, y2 = layer(x), layer(x)
    assert torch.equal(y1, y2)
    assert 0.0 < layer.last_dropped_token_fraction < 1.0
    idx, w, _ = layer.router(x)
    keep = ~compute_capacity_drop_mask(idx, 4, layer.capacity(64))
    want = experts_reference(x, idx, w, layer.w13, layer.w2, 0, keep)
    assert torch.allclose(y1, want, atol=1e-5)
    free = DistributedMoELayer(16, 32, 4, 2)
    free(x)
    assert free.last_dropped_token_fraction == 0.0


def test_topology_ownership_and_coordinates():
    for ep in (1, 2, 3, 4):
        seen = []
        for r in range(ep):
            t = ParallelTopology(world_size=ep, rank=r, dp_size=1, ep_size=ep)
            seen += t.experts_on_this_rank(10)
        assert seen == list(range(10))
    t = ParallelTopology(world_size=4, rank=1, dp_size=1, ep_size=4)
    assert t.experts_on_this_rank(10) == [3, 4, 5]
    t = ParallelTopology(world_size=16, rank=13, dp_size=2, ep_size=2, tp_size=2, pp_size=2)
    assert (t.dp_rank, t.tp_rank, t.pp_rank, t.ep_rank) == (1, 1, 0, 1)
    assert t.rank_of(1, 1, 0, 1) == 13
    t.validate_world_size()
    with pytest.raises(ValueError):
        ParallelTopology(world_size=7, rank=0, dp_size=2, ep_size=2).validate_world_size()
    c = ParallelTopology(world_size=8, rank=5, dp_size=2, ep_size=2, tp_size=2, pp_size=2, ep_from_dp=True)
    assert (c.dp_rank, c.tp_rank, c.pp_rank, c.ep_rank) == (1, 0, 1, 1)
    assert c.axis_ranks("ep") == [1, 5] and c.axis_ranks("tp") == [5, 7] and c.axis_ranks("pp") == [4, 5]
    assert build_topology(8, 8, 2, 2, device_type="cpu").world_size == 1  # degenerate without a process group


def test_expert_to_rank_round_trip():
    topo = ParallelTopology(world_size=3, rank=0, dp_size=1, ep_size=3)
    layer = DistributedMoELayer(8, 16, 10, 2, topology=topo)
    for r in range(3):
        for e in topo.experts_on_rank(10, r):
            assert layer._expert_to_rank(e) == r
    # tensor in, tensor of ranks out (the reference's calling convention, pkg/distributed/moe_layer.py:362-389)
    ids = torch.arange(10).view(2, 5)
    ranks = layer._expert_to_rank(ids)
    assert ranks.shape == ids.shape and ranks.dtype == torch.int64
    assert ranks.flatten().tolist() == [layer._expert_to_rank(int(e)) for e in ids.flatten()]


def test_tp1_linears_equal_nn_linear():
    torch.manual_seed(4)
    col, row = ColumnParallelLinear(16, 24), RowParallelLinear(24, 16)
    x = torch.randn(3, 5, 16)
    assert torch.allclose(col(x), F.linear(x, col.weight, col.bias))
    h = col(x)
    assert torch.allclose(row(h), F.linear(h, row.weight, row.bias))
    assert col.weight.shape == (24, 16) and row.weight.shape == (16, 24)
    with pytest.raises(ValueError):
        ColumnParallelLinear(16, 25, topology=ParallelTopology(2, 0, 1, 1, tp_size=2))


def test_sequence_parallel_identity_at_tp1():
    x = torch.randn(2, 8, 16)
    topo = ParallelTopology(1, 0, 1, 1)
    assert torch.equal(scatter_to_sequence_parallel(x, topo), x)
    assert torch.equal(gather_from_sequence_parallel(x, topo), x)
    w = torch.randn(4, 16)
    assert torch.allclose(scatter_to_sequence_parallel(x, topo, next_weight=w), F.linear(x, w))
