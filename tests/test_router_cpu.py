"""Router numerics on the PyTorch path: oracle agreement, analytic backward, invariants, edge cases, interface.
Test strategy of the reference's tests/test_kernels.py, test_kernels_numerics.py, test_router.py and
test_routing_quality.py."""

import math

import pytest
import torch

from composed_mixture_of_experts_engine_b200.ops.moe_router import (MIN_TRITON_DIM, TRITON_AVAILABLE, MoERouter,
                                                                    MoERouterAutograd, MoERouterFunction,
                                                                    _compute_load_imbalance, _compute_router_z_loss,
                                                                    _reference_backward_fp64, _reference_route_fp64,
                                                                    _should_use_triton, moe_topk_route)
from composed_mixture_of_experts_engine_b200.parallel.router import MoERouterInterface, RouterStats

pytestmark = pytest.mark.cpu


@pytest.mark.parametrize("N,H,E,K", [(64, 32, 8, 2), (100, 48, 16, 4), (33, 16, 4, 1), (20, 24, 6, 6)])
def test_route_matches_oracle(N, H, E, K):
    torch.manual_seed(0)
    x, w = torch.randn(N, H), torch.randn(H, E) / math.sqrt(H)
    idx, wt = moe_topk_route(x, w, K)
    ridx, rw, _ = _reference_route_fp64(x, w, K)
    assert idx.dtype == torch.int64 and torch.equal(idx, ridx)
    assert torch.allclose(wt, rw, atol=1e-5, rtol=1e-5)
    assert torch.allclose(wt.sum(-1), torch.ones(N), atol=1e-5)
    assert all(len(set(r.tolist())) == K for r in idx)  # distinct experts per token
    assert int(torch.bincount(idx.flatten(), minlength=E).sum()) == N * K  # conservation


def test_backward_matches_autograd():
    torch.manual_seed(1)
    N, H, E, K = 40, 32, 8, 2
    x = torch.randn(N, H, dtype=torch.float64, requires_grad=True)
    w = (torch.randn(H, E, dtype=torch.float64) / math.sqrt(H)).requires_grad_(True)
    gw = torch.randn(N, K, dtype=torch.float64)
    idx, wt = MoERouterFunction.apply(x, w, K, False, None)
    (wt * gw).sum().backward()
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    p = torch.softmax(x2 @ w2, -1)
    v, i2 = torch.topk(p, K, -1)
    ((v / v.sum(-1, keepdim=True)) * gw).sum().backward()
    assert torch.equal(idx, i2)
    assert torch.allclose(x.grad, x2.grad, atol=1e-9) and torch.allclose(w.grad, w2.grad, atol=1e-9)
    gl = _reference_backward_fp64((x2 @ w2).detach(), idx, gw, K, E)
    assert torch.allclose(gl @ w2.detach().t(), x2.grad, atol=1e-9)


def test_determinism_and_3d_input():
    torch.manual_seed(2)
    x, w = torch.randn(2, 10, 16), torch.randn(16, 8)
    a = moe_topk_route(x, w, 2)
    b = moe_topk_route(x.reshape(20, 16), w, 2)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    with pytest.raises(ValueError):
        moe_topk_route(torch.randn(16), w, 2)
    with pytest.raises(ValueError):
        moe_topk_route(x, w, 9)


def test_edge_cases():
    w = torch.randn(16, 4)
    idx, wt = moe_topk_route(torch.randn(1, 16), w, 1)
    assert idx.shape == (1, 1) and torch.allclose(wt, torch.ones(1, 1))
    idx, wt = moe_topk_route(torch.randn(5, 16), w, 4)  # K == E
    assert sorted(idx[0].tolist()) == [0, 1, 2, 3]
    big = moe_topk_route(torch.randn(8, 16) * 10, w * 10, 2)[1]
    assert torch.isfinite(big).all()


def test_api_constants():
    assert MoERouterAutograd is MoERouterFunction and TRITON_AVAILABLE is False and MIN_TRITON_DIM == 16
    assert _should_use_triton(torch.randn(64, 32), torch.randn(32, 16), False) is False  # CPU tensors


def test_metrics_closed_forms():
    assert _compute_load_imbalance(torch.tensor([4, 4, 4, 4])) == pytest.approx(1.0)
    assert _compute_load_imbalance(torch.tensor([8, 0, 0, 0])) == pytest.approx(4.0)
    assert _compute_load_imbalance(torch.zeros(4)) == 1.0
    logits = torch.zeros(5, 8)
    assert _compute_router_z_loss(logits) == pytest.approx(math.log(8) ** 2, rel=1e-6)


def test_module_forward_profile_and_grads():
    torch.manual_seed(3)
    r = MoERouter(32, 8, top_k=2)
    assert r.gate_w.shape == (32, 8)
    x = torch.randn(50, 32, requires_grad=True)
    idx, w, cnt = r(x)
    assert idx.shape == (50, 2) and cnt.dtype == torch.int64 and int(cnt.sum()) == 100
    (w.sum() + r.last_aux_loss + 1e-3 * r.last_z_loss).backward()
    assert r.gate_w.grad is not None and torch.isfinite(r.gate_w.grad).all() and x.grad.abs().sum() > 0
    p = r.last_profile
    assert p.used_triton is False and p.used_fused_kernel is False
    assert p.sram_bytes_per_block == 128 * 64 * 2 + 64 * 64 * 2  # one stage of the fused kernel's tiles
    assert p.tokens_per_expert_mean == pytest.approx(100 / 8)
    assert p.expert_load_imbalance == pytest.approx(float(cnt.max()) / (100 / 8))
    assert p.router_z_loss == pytest.approx(_compute_router_z_loss(r._last_logits), rel=1e-4)
    f = cnt.double() / 100
    probs = torch.softmax(x.detach().double() @ r.gate_w.detach().double(), -1)
    assert float(r.last_aux_loss) == pytest.approx(8 * float((f * probs.mean(0)).sum()), rel=1e-5)
    with pytest.raises(ValueError):
        MoERouter(32, 4, top_k=5)


def test_bias_path():
    r = MoERouter(16, 4, top_k=2, bias=True)
    with torch.no_grad():
        r.bias[3] = 100.0
    idx, w, cnt = r(torch.randn(10, 16))
    assert (idx[:, 0] == 3).all()


def test_interface_validation_and_budget():
    ri = MoERouterInterface(32, 8, 2, capacity_factor=1.25)
    stats = ri(torch.randn(64, 32))
    assert isinstance(stats, RouterStats) and stats.expert_indices.shape == (64, 2)
    assert int(stats.dispatch_counts.sum()) == 128 and stats.used_triton is False
    with pytest.raises(ValueError):
        ri(torch.randn(2, 32, 32))
    with pytest.raises(ValueError):
        ri(torch.randn(64, 16))
    for n, want in [(64, 20), (100, 32), (1, 1), (1000, 313)]:
        assert ri.capacity_budget(n) == want == math.ceil(1.25 * n * 2 / 8)
    with pytest.raises(ValueError):
        MoERouterInterface(32, 4, 8)
    with pytest.warns(UserWarning, match="silently drop tokens"):
        MoERouterInterface(32, 4, 2, capacity_factor=0.9)
    torch.randn(4, 32)
    stats.combine_weights.sum()
    x = torch.randn(16, 32, requires_grad=True)
    ri(x).combine_weights.sum().backward()
    assert ri._kernel_router.gate_w.grad is not None
