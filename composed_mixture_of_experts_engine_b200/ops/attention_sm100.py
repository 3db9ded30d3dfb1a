"""Hand-written causal attention for B200: ``csrc/attention.cu`` (tcgen05.mma into TMEM, TMA tiles of the packed
projection, softmax with one thread per row out of TMEM; forward and backward, grouped-query heads).

The kernels work on the packed projection ``qkv`` [B, S, nh + 2 nkv, hd] (q heads, k heads, v heads; bf16,
contiguous) with S a multiple of 128 and hd 64 or 128.  ``CMOE_ATTN_SM100=1`` routes
``ops.functional.rope_causal_attention`` and ``ops.attention.causal_attention`` through them; without it the
library path (cuDNN's fused attention through ``scaled_dot_product_attention``) runs.  The reference has no
attention operator at all (pkg/models/moe.py:148-186).
"""

from __future__ import annotations

import os
from typing import Tuple

import torch

from . import _ext
from . import kernels as _k


def enabled() -> bool:
    return os.environ.get("CMOE_ATTN_SM100", "0") == "1"


def shape_supported(S: int, nh: int, nkv: int, hd: int) -> bool:
    return S > 0 and S % 128 == 0 and hd in (64, 128) and nkv > 0 and nh % nkv == 0


def packed_supported(qkv: torch.Tensor, nh: int, nkv: int) -> bool:
    return (
        qkv.is_cuda
        and qkv.dtype == torch.bfloat16
        and qkv.dim() == 4
        and qkv.is_contiguous()
        and qkv.shape[2] == nh + 2 * nkv
        and shape_supported(qkv.shape[1], nh, nkv, qkv.shape[3])
    )


def forward_packed(qkv: torch.Tensor, nh: int, nkv: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (out bf16 [B, S, nh, hd], lse fp32 [B, nh, S])."""
    B, S, _, hd = qkv.shape
    out = torch.empty(B, S, nh, hd, device=qkv.device, dtype=torch.bfloat16)
    lse = torch.empty(B, nh, S, device=qkv.device, dtype=torch.float32)
    _ext.ext().attention_fwd(qkv, nh, nkv, out, lse, _k.status_word(qkv.device), 0)
    return out, lse


def backward_packed(
    qkv: torch.Tensor, nh: int, nkv: int, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (dq fp32 [B, S, nh, hd], dk bf16 [B, S, nkv, hd], dv bf16 [B, S, nkv, hd])."""
    B, S, _, hd = qkv.shape
    dq = torch.zeros(B, S, nh, hd, device=qkv.device, dtype=torch.float32)
    dk = torch.empty(B, S, nkv, hd, device=qkv.device, dtype=torch.bfloat16)
    dv = torch.empty(B, S, nkv, hd, device=qkv.device, dtype=torch.bfloat16)
    delta = torch.empty(B, nh, S, device=qkv.device, dtype=torch.float32)
    _ext.ext().attention_bwd(qkv, nh, nkv, out, dout.contiguous(), lse, delta, dq, dk, dv,
                             _k.status_word(qkv.device), 0)
    return dq, dk, dv


class _PackedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, nh, nkv):
        out, lse = forward_packed(qkv, nh, nkv)
        ctx.save_for_backward(qkv, out, lse)
        ctx.heads = (nh, nkv)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        nh, nkv = ctx.heads
        dq, dk, dv = backward_packed(qkv, nh, nkv, out, dout, lse)
        return torch.cat([dq.to(torch.bfloat16), dk, dv], dim=2), None, None


def packed_causal_attention(qkv: torch.Tensor, nh: int, nkv: int) -> torch.Tensor:
    """Differentiable causal attention on a packed, already rotated projection."""
    return _PackedAttentionFn.apply(qkv, nh, nkv)


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    if not (enabled() and q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4):
        return False
    return k.shape == v.shape and shape_supported(q.shape[1], q.shape[2], k.shape[2], q.shape[3])


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [B,S,nh,hd], k/v [B,S,nkv,hd] -> [B,S,nh,hd]; packs the three into one buffer first."""
    return packed_causal_attention(torch.cat([q, k, v], dim=2), q.shape[2], k.shape[2])
