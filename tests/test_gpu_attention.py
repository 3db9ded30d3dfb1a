"""Numerics of the hand-written tcgen05 attention kernels (csrc/attention.cu) against the fp32 PyTorch restatement
of causal grouped-query attention under plain autograd.

The reference has no attention operator (pkg/models/moe.py:148-186), so the oracle is this package's own
``attention_reference``.
"""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, S, nh, nkv, hd
    (1, 384, 4, 2, 128),   # grouped-query, three key tiles, off-diagonal and diagonal tiles
    (2, 256, 2, 2, 64),    # one 64-column block per head
    (1, 128, 2, 1, 128),   # a single (diagonal) tile
    (1, 512, 4, 2, 128),   # S a multiple of 256 at hd 128: the two-query-tile forward kernel
]


def _reference(qkv, go, nh, nkv):
    from composed_mixture_of_experts_engine_b200.ops.attention import attention_reference

    q = qkv[:, :, :nh].float().requires_grad_()
    k = qkv[:, :, nh: nh + nkv].float().requires_grad_()
    v = qkv[:, :, nh + nkv:].float().requires_grad_()
    out = attention_reference(q, k, v)
    out.backward(go.float())
    S, hd = qkv.shape[1], qkv.shape[3]
    qf = q.detach().permute(0, 2, 1, 3)
    kf = k.detach().permute(0, 2, 1, 3).repeat_interleave(nh // nkv, 1)
    scores = (qf @ kf.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    lse = torch.logsumexp(scores.masked_fill(~mask, float("-inf")), -1)
    return out.detach(), lse, q.grad, k.grad, v.grad


@pytest.mark.parametrize("B,S,nh,nkv,hd", SHAPES)
def test_attention_kernels_match_fp32_restatement(B, S, nh, nkv, hd):
    from composed_mixture_of_experts_engine_b200.ops import attention_sm100 as A
    from composed_mixture_of_experts_engine_b200.ops import kernels

    torch.manual_seed(0)
    dev = torch.device("cuda")
    qkv = torch.randn(B, S, nh + 2 * nkv, hd, device=dev).to(torch.bfloat16)
    go = torch.randn(B, S, nh, hd, device=dev).to(torch.bfloat16)
    ref, lse_ref, dq_ref, dk_ref, dv_ref = _reference(qkv, go, nh, nkv)

    assert A.packed_supported(qkv, nh, nkv)
    out, lse = A.forward_packed(qkv, nh, nkv)
    torch.cuda.synchronize()
    kernels.check_status(dev)
    assert (out.float() - ref).abs().max() < 3e-2
    assert (lse - lse_ref).abs().max() < 1e-3

    dq, dk, dv = A.backward_packed(qkv, nh, nkv, out, go, lse)
    torch.cuda.synchronize()
    kernels.check_status(dev)
    for got, want in ((dq, dq_ref), (dk.float(), dk_ref), (dv.float(), dv_ref)):
        assert (got - want).norm() / want.norm() < 2e-2
        assert (got - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max()))


def test_packed_rope_attention_runs_on_the_sm100_kernels(monkeypatch):
    """With CMOE_ATTN_SM100=1 the packed RoPE + attention op of the decoder goes through the hand-written kernels
    and agrees with the default (library attention) path, values and input gradient."""
    from composed_mixture_of_experts_engine_b200.ops import functional as OF

    torch.manual_seed(5)
    B, S, nh, nkv, hd = 2, 256, 4, 2, 128
    heads = nh + 2 * nkv
    cos, sin = OF.rope_tables(S, hd, 10000.0, torch.device("cuda"))
    base = torch.randn(B, S, heads, hd, device="cuda").to(torch.bfloat16)
    go = torch.randn(B, S, nh, hd, device="cuda").to(torch.bfloat16)

    def run():
        x = base.clone().requires_grad_()
        out = OF.rope_causal_attention(x * 1.0, cos, sin, nh, nkv)  # x * 1.0: the op consumes its input buffer
        out.backward(go)
        return out.float(), x.grad.float()

    monkeypatch.setenv("CMOE_ATTN_SM100", "0")
    want, gwant = run()
    monkeypatch.setenv("CMOE_ATTN_SM100", "1")
    got, ggot = run()
    assert (got - want).norm() / want.norm() < 2e-2
    assert (ggot - gwant).norm() / gwant.norm() < 3e-2


def test_unsupported_shapes_fall_back(monkeypatch):
    from composed_mixture_of_experts_engine_b200.ops import attention_sm100 as A

    monkeypatch.setenv("CMOE_ATTN_SM100", "1")
    q = torch.randn(1, 96, 2, 64, device="cuda", dtype=torch.bfloat16)  # S not a multiple of 128
    assert not A.supported(q, q, q)
    assert not A.shape_supported(256, 4, 3, 128) and not A.shape_supported(256, 4, 2, 96)
    assert A.shape_supported(4096, 16, 16, 128) and A.shape_supported(4096, 32, 8, 128)
