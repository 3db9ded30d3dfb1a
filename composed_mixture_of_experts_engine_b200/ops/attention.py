"""Causal self-attention with grouped-query support.

``causal_attention(q, k, v)`` takes q [B,S,nh,hd] and k/v [B,S,nkv,hd] and returns [B,S,nh,hd].
The PyTorch restatement (fp32 softmax) is the CPU path and the oracle of the GPU tests.  The
reference has no attention operator at all (pkg/models/moe.py:148-186); this op exists because the
benchmark configurations name heads, GQA and RoPE.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    B, S, nh, hd = q.shape
    nkv = k.shape[2]
    rep = nh // nkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    scores = qf @ kf.transpose(-1, -2) / math.sqrt(hd)
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    out = torch.softmax(scores, dim=-1) @ vf
    return out.permute(0, 2, 1, 3).to(q.dtype).contiguous()


def _sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    nh, nkv = q.shape[2], k.shape[2]
    qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    if nkv != nh:
        kt = kt.repeat_interleave(nh // nkv, dim=1)
        vt = vt.repeat_interleave(nh // nkv, dim=1)
    out = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    return out.permute(0, 2, 1, 3).contiguous()


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    if q.is_cuda and q.dtype == torch.bfloat16:
        from . import attention_sm100

        if attention_sm100.supported(q, k, v):
            return attention_sm100.causal_attention(q, k, v)
    return _sdpa(q, k, v)
