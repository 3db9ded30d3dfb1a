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


_NATIVE_GQA = {"cuda": None}  # None: not probed yet; True / False: whether a fused kernel takes grouped K / V


def sdpa_grouped(qt: torch.Tensor, kt: torch.Tensor, vt: torch.Tensor) -> torch.Tensor:
    """Causal ``scaled_dot_product_attention`` on [B, heads, S, hd] tensors whose K / V carry fewer heads than Q.

    On CUDA the fused library kernels read the shared K / V heads in place (``enable_gqa=True``) instead of from
    copies repeated ``nh / nkv`` times.  Whether the installed PyTorch has a fused kernel for that is found out on
    the first call (restricted to the fused backends, so that a silent fall-back to the unfused math kernel cannot
    happen); if not, K / V are repeated as before."""
    nh, nkv = qt.shape[1], kt.shape[1]
    if nkv == nh:
        return F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    if qt.is_cuda and _NATIVE_GQA["cuda"] is not False:
        try:
            from torch.nn.attention import SDPBackend, sdpa_kernel

            with sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION]):
                out = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True)
            _NATIVE_GQA["cuda"] = True
            return out
        except Exception:
            if _NATIVE_GQA["cuda"] is True:
                raise
            _NATIVE_GQA["cuda"] = False
    rep = nh // nkv
    return F.scaled_dot_product_attention(qt, kt.repeat_interleave(rep, dim=1), vt.repeat_interleave(rep, dim=1),
                                          is_causal=True)


def _sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    return sdpa_grouped(qt, kt, vt).permute(0, 2, 1, 3).contiguous()


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    if q.is_cuda and q.dtype == torch.bfloat16:
        from . import attention_sm100

        if attention_sm100.supported(q, k, v):
            return attention_sm100.causal_attention(q, k, v)
    return _sdpa(q, k, v)
