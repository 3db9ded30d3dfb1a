"""Differentiable ops of the model, each with one CUDA path (the sm_100a kernels) and one PyTorch path.

The PyTorch path is what runs on CPU (gloo tests, the fp32 smoke config) and what the GPU numerics
tests compare against; on a CUDA device with bf16 tensors the kernels are the only path.  Reference
counterparts: RMSNorm (pkg/models/moe.py:63-86), the expert FFN and dispatch/combine of
``DistributedMoELayer.forward`` (pkg/distributed/moe_layer.py:264-360), cross-entropy (train.py:297-303).
RoPE and attention are additions (the reference model has neither).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _ext, kernels
from . import attention_sm100 as _attn_sm100
from .kernels import EPI_SWIGLU_BWD, EPI_SWIGLU_FWD, GEMM_GROUPED_K, GEMM_GROUPED_M, MoEPlan


def force_library() -> bool:
    """``CMOE_FORCE_LIBRARY=1``: every differentiable op takes its PyTorch path even on a B200 (the library arm of
    the benchmarks: cuBLAS / cuDNN / eager kernels through PyTorch, nothing of this package's device code)."""
    import os

    return os.environ.get("CMOE_FORCE_LIBRARY", "0") == "1"


def on_device_path(*tensors: torch.Tensor) -> bool:
    """True when the sm_100a kernels handle these tensors (CUDA + bf16)."""
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors) and not force_library()


# ------------------------------------------------------------------------------------------ RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], device=x.device, dtype=torch.float32)
        _ext.ext().rmsnorm_fwd(xc, weight, y, rstd, eps)
        ctx.save_for_backward(xc, weight, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        dx = torch.empty_like(x)
        dw = torch.zeros(weight.shape, device=x.device, dtype=torch.float32)
        _ext.ext().rmsnorm_bwd(dy.contiguous(), x, weight, rstd, dx, dw)
        return dx, dw.to(weight.dtype), None


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if on_device_path(x, weight) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192:
        return _RMSNormFn.apply(x, weight, eps)
    return rmsnorm_reference(x, weight, eps)


# ------------------------------------------------------------------------------------------ dense linear
def rows_for_tma(t: torch.Tensor) -> torch.Tensor:
    """``t`` [rows, cols] as a contiguous tensor whose first element sits on a 16-byte boundary (what a TMA
    tensor map needs); a copy only when the view it was given does not already qualify."""
    if not t.is_contiguous():
        return t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


class _LinearFn(torch.autograd.Function):
    """``y = x @ W^T`` on the two-SM tcgen05 GEMM: forward K-major x K-major, input gradient with W read
    N-major (no transposed copy), weight gradient as a contraction over the rows whose fp32 result is added into
    ``W.main_grad`` by the kernel's TMA reduce-add epilogue when the optimizer gave the parameter one."""

    @staticmethod
    def forward(ctx, x, weight):
        K = x.shape[-1]
        x2 = rows_for_tma(x.reshape(-1, K))
        y = kernels.linear_nt(x2, weight)
        ctx.save_for_backward(x2, weight)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        N, K = weight.shape
        dy2 = rows_for_tma(dy.reshape(-1, N))
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = kernels.linear_nn(dy2, weight).view(*dy.shape[:-1], K)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None:
                kernels.linear_tn_acc(dy2, x2, main)
            else:
                dw = kernels.linear_tn(dy2, x2).to(weight.dtype)
        return dx, dw


def linear_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The tcgen05 GEMM takes this projection: CUDA bf16, feature counts that are multiples of 8 (TMA rows start
    on 16-byte boundaries), a contiguous weight whose storage starts on a 16-byte boundary."""
    return (on_device_path(x, weight) and weight.dim() == 2 and weight.is_contiguous()
            and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0 and weight.data_ptr() % 16 == 0
            and x.shape[-1] == weight.shape[1] and x.numel() > 0)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight^T (+ bias)`` with ``weight`` [out, in] (the ``nn.Linear`` contraction).  Reference counterpart:
    the ``F.linear`` calls of pkg/distributed/tensor_parallel.py:121,197 and pkg/models/moe.py:186 (cuBLAS there)."""
    if linear_supported(x, weight):
        y = _LinearFn.apply(x, weight)
        return y if bias is None else y + bias
    return F.linear(x, weight, bias)


# ------------------------------------------------------------------------------------------ RoPE
def rope_tables(seq_len: int, head_dim: int, theta: float, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


class _RopeFn(torch.autograd.Function):
    """Rotates the first ``n_rot_heads`` heads of ``t`` [rows, heads, head_dim] in place."""

    @staticmethod
    def forward(ctx, t, cos, sin, seq, n_rot_heads):
        view = t[:, :n_rot_heads]
        _ext.ext().rope(view, cos, sin, seq, False)
        ctx.save_for_backward(cos, sin)
        ctx.seq, ctx.n_rot = seq, n_rot_heads
        ctx.mark_dirty(t)
        return t

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        g = g.contiguous().clone()
        _ext.ext().rope(g[:, : ctx.n_rot], cos, sin, ctx.seq, True)
        return g, None, None, None, None


def rope_reference(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq: int, n_rot_heads: int) -> torch.Tensor:
    rows, heads, hd = t.shape
    pos = torch.arange(rows, device=t.device) % seq
    c = cos[pos][:, None, :].to(torch.float32)
    s = sin[pos][:, None, :].to(torch.float32)
    rot = t[:, :n_rot_heads].float()
    a, b = rot[..., : hd // 2], rot[..., hd // 2:]
    out = torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(t.dtype)
    return torch.cat([out, t[:, n_rot_heads:]], dim=1)


def rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq: int, n_rot_heads: int) -> torch.Tensor:
    """Rotary embedding on heads [0, n_rot_heads) of ``t`` [rows, heads, head_dim]; row r sits at position r % seq."""
    if on_device_path(t) and t.shape[-1] % 16 == 0 and t.is_contiguous():
        return _RopeFn.apply(t, cos, sin, seq, n_rot_heads)
    return rope_reference(t, cos, sin, seq, n_rot_heads)


# ------------------------------------------------------------------------------------------ attention
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [B,S,nh,hd], k/v [B,S,nkv,hd] -> [B,S,nh,hd], causal, grouped-query when nkv < nh."""
    from . import attention as _attn

    return _attn.causal_attention(q, k, v)


class _RopeAttentionFn(torch.autograd.Function):
    """RoPE + causal attention on a packed projection ``qkv`` [B, S, nh + 2 nkv, hd].

    The rotation runs in place on ``qkv`` (the caller hands over the projection's output and must not read it
    afterwards), the attention kernel reads q / k / v as strided views of the packed buffer, and the backward
    packs dq / dk / dv into one gradient buffer and un-rotates the q and k heads in the same pass.  This replaces the
    slice / zero-fill / accumulate chain autograd would build around three views of one tensor (three zero
    fills and two adds of the full packed size per layer)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, nh, nkv):
        B, S, heads, hd = qkv.shape
        _ext.ext().rope(qkv.view(B * S, heads, hd)[:, : nh + nkv], cos, sin, S, False)
        t = qkv.detach()
        ctx.dims = (B, S, heads, hd, nh, nkv)
        if _attn_sm100.enabled() and _attn_sm100.packed_supported(t, nh, nkv):
            # hand-written tcgen05 kernels on the packed buffer; the backward needs the rotated projection,
            # the output and the row log-sum-exps
            out, lse = _attn_sm100.forward_packed(t, nh, nkv)
            ctx.inner = (t, out, lse)
            ctx.sm100 = True
            ctx.save_for_backward(cos, sin)
            return out
        ctx.sm100 = False
        with torch.enable_grad():
            q = t[:, :, :nh].permute(0, 2, 1, 3).requires_grad_()
            k = t[:, :, nh: nh + nkv].permute(0, 2, 1, 3).requires_grad_()
            v = t[:, :, nh + nkv:].permute(0, 2, 1, 3).requires_grad_()
            from .attention import sdpa_grouped

            out = sdpa_grouped(q, k, v)  # grouped K / V are read in place where the library has a fused kernel for it
        ctx.inner = (q, k, v, out)
        ctx.save_for_backward(cos, sin)
        ctx.dims = (B, S, heads, hd, nh, nkv)
        return out.detach().permute(0, 2, 1, 3).contiguous()

    @staticmethod
    def backward(ctx, go):
        cos, sin = ctx.saved_tensors
        B, S, heads, hd, nh, nkv = ctx.dims
        dqkv = torch.empty(B, S, heads, hd, device=go.device, dtype=go.dtype)
        if ctx.sm100:
            t, out, lse = ctx.inner
            ctx.inner = None
            dq32, dk, dv = _attn_sm100.backward_packed(t, nh, nkv, out, go, lse)
            _ext.ext().qkv_grad_pack(dq32.to(torch.bfloat16).permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3),
                                     dv.permute(0, 2, 1, 3), dqkv, cos, sin)
            return dqkv, None, None, None, None
        q, k, v, out = ctx.inner
        ctx.inner = None
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), go.permute(0, 2, 1, 3))
        if all(t.stride(3) == 1 and all(st % 8 == 0 for st in t.stride()[:3]) for t in (dq, dk, dv)):
            # one pass: pack the three gradients and undo the rotation of the q and k heads on the way
            _ext.ext().qkv_grad_pack(dq, dk, dv, dqkv, cos, sin)
        else:
            dqkv[:, :, :nh].copy_(dq.permute(0, 2, 1, 3))
            dqkv[:, :, nh: nh + nkv].copy_(dk.permute(0, 2, 1, 3))
            dqkv[:, :, nh + nkv:].copy_(dv.permute(0, 2, 1, 3))
            _ext.ext().rope(dqkv.view(B * S, heads, hd)[:, : nh + nkv], cos, sin, S, True)
        return dqkv, None, None, None, None


def rope_causal_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nh: int, nkv: int) -> torch.Tensor:
    """``qkv`` [B, S, nh + 2 nkv, hd] (q heads, then k heads, then v heads) -> attention output [B, S, nh, hd] with
    rotary embedding on q and k.  On the device path ``qkv`` is consumed (rotated in place)."""
    B, S, heads, hd = qkv.shape
    if on_device_path(qkv) and hd % 16 == 0 and qkv.is_contiguous():
        return _RopeAttentionFn.apply(qkv, cos, sin, nh, nkv)
    t = rope(qkv.reshape(B * S, heads, hd), cos, sin, S, nh + nkv).view(B, S, heads, hd)
    return causal_attention(t[:, :, :nh], t[:, :, nh: nh + nkv], t[:, :, nh + nkv:])


# ------------------------------------------------------------------------------------------ cross-entropy
class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, scale):
        loss = torch.zeros(1, device=logits.device, dtype=torch.float32)
        _ext.ext().cross_entropy(logits, targets, loss, scale)
        ctx.save_for_backward(logits)  # now holds d(loss)/d(logits)
        return loss[0] * scale

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return grad * g.to(grad.dtype), None, None


def cross_entropy_sum_scaled(logits: torch.Tensor, targets: torch.Tensor, scale: float) -> torch.Tensor:
    """``scale * sum_rows CE(logits, targets)``.  On the device path the logits buffer is consumed:
    it is overwritten with the gradient, so the caller must not use it afterwards."""
    if on_device_path(logits) and logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        return _CrossEntropyFn.apply(logits, targets, scale)
    return F.cross_entropy(logits.float(), targets, reduction="sum", ignore_index=-100) * scale


# ------------------------------------------------------------------------------------------ expert FFN
def experts_reference(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                      expert_lo: int = 0, keep: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y_t = sum_k w[t,k] * Expert_{idx[t,k]}(x_t) for the experts [expert_lo, expert_lo + E_local) held in
    ``w13`` [E_local, 2F, H] (gate rows then up rows) and ``w2`` [E_local, H, F].  Plain PyTorch, any dtype."""
    N, H = x.shape
    E_local, twoF, _ = w13.shape
    Fdim = twoF // 2
    y = torch.zeros(N, H, dtype=torch.float32, device=x.device)
    for e in range(E_local):
        mask = idx == (e + expert_lo)
        if keep is not None:
            mask = mask & keep
        tok, slot = mask.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        g = xe @ w13[e, :Fdim].t()
        u = xe @ w13[e, Fdim:].t()
        out = (F.silu(g) * u) @ w2[e].t()
        y.index_add_(0, tok, out.float() * w[tok, slot].float()[:, None])
    return y.to(x.dtype)


def _weight_grad(a: torch.Tensor, b: torch.Tensor, param: torch.Tensor, M: int, N: int, plan: MoEPlan):
    """dW[e] = a[rows_e, :M]^T @ b[rows_e, :N]; accumulated into ``param.main_grad`` (fp32) when present."""
    E = plan.n_local
    main = getattr(param, "main_grad", None)
    if main is not None:
        kernels.gemm(a, b, main.view(E, M, N), mode=GEMM_GROUPED_K, M=M, N=N, a_mn=True, b_mn=True, groups=E,
                     group_offsets=plan.group_offsets, d_group_stride=M * N, accumulate=True)
        return None
    out = torch.empty(E, M, N, device=a.device, dtype=torch.float32)
    kernels.gemm(a, b, out, mode=GEMM_GROUPED_K, M=M, N=N, a_mn=True, b_mn=True, groups=E,
                 group_offsets=plan.group_offsets, d_group_stride=M * N)
    return out.to(param.dtype)


def grouped_swiglu_forward(xp: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, plan: MoEPlan,
                           ready: Optional[dict] = None, yp_out: Optional[torch.Tensor] = None,
                           pull: Optional[dict] = None, scatter: Optional[dict] = None):
    """(hact, gu, yp) for expert-sorted rows ``xp`` [cap_rows, H].  With ``pull`` (src_ptrs, slots_per_src, pull_K,
    ld_src) the first GEMM fills ``xp`` itself from the ranks' token buffers while it runs (fused dispatch)."""
    E, twoF, H = w13.shape
    Fdim = twoF // 2
    dev = xp.device
    hact = torch.empty(plan.cap_rows, Fdim, device=dev, dtype=torch.bfloat16)
    gu = torch.empty(plan.cap_rows, twoF, device=dev, dtype=torch.bfloat16)
    yp = None
    if scatter is None:
        yp = yp_out if yp_out is not None else torch.empty(plan.cap_rows, H, device=dev, dtype=torch.bfloat16)
    kw = ready or {}
    if pull is not None:
        kernels.gemm_pull(xp, w13.view(E * twoF, H), hact, plan, epilogue=EPI_SWIGLU_FWD, N=Fdim, K=H, groups=E,
                          b_group_rows=twoF, split_n=Fdim, aux_out=gu, **pull)
    else:
        kernels.gemm(xp, w13.view(E * twoF, H), hact, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_FWD, N=Fdim, K=H,
                     groups=E, b_group_rows=twoF, split_n=Fdim, tile_group=plan.tile_group,
                     num_m_tiles=plan.num_m_tiles, max_m_tiles=plan.max_m_tiles, aux_out=gu, **kw)
    if scatter is not None:  # the result rows go straight to the ranks that own the tokens (fused combine push)
        kernels.gemm_scatter(hact, w2.view(E * H, Fdim), N=H, K=Fdim, plan=plan, groups=E, b_group_rows=H, **scatter)
    else:
        kernels.gemm(hact, w2.view(E * H, Fdim), yp, mode=GEMM_GROUPED_M, N=H, K=Fdim, groups=E, b_group_rows=H,
                     tile_group=plan.tile_group, num_m_tiles=plan.num_m_tiles, max_m_tiles=plan.max_m_tiles)
    return hact, gu, yp


def grouped_swiglu_backward(dyp: torch.Tensor, xp: torch.Tensor, hact: torch.Tensor, gu: torch.Tensor,
                            w13: torch.Tensor, w2: torch.Tensor, plan: MoEPlan, need_dx: bool = True,
                            dxp_out: Optional[torch.Tensor] = None, pull: Optional[dict] = None,
                            scatter: Optional[dict] = None):
    """(dxp, dW13, dW2) of the grouped SwiGLU FFN; weight gradients go to ``main_grad`` when the parameters have one."""
    E, twoF, H = w13.shape
    Fdim = twoF // 2
    dgu = torch.empty_like(gu)
    if pull is not None:  # dyp is filled from the ranks' dy buffers (times the gate weights) by the kernel itself
        kernels.gemm_pull(dyp, w2.view(E * H, Fdim), dgu, plan, epilogue=EPI_SWIGLU_BWD, N=Fdim, K=H, b_mn=True,
                          groups=E, b_group_rows=H, aux_in=gu, **pull)
    else:
        kernels.gemm(dyp, w2.view(E * H, Fdim), dgu, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_BWD, N=Fdim, K=H,
                     b_mn=True, groups=E, b_group_rows=H, tile_group=plan.tile_group, num_m_tiles=plan.num_m_tiles,
                     max_m_tiles=plan.max_m_tiles, aux_in=gu)
    dxp = None
    if need_dx:
        if scatter is not None:  # dX rows are pushed to the token owners by the epilogue
            kernels.gemm_scatter(dgu, w13.view(E * twoF, H), N=H, K=twoF, plan=plan, groups=E, b_group_rows=twoF,
                                 b_mn=True, **scatter)
        else:
            dxp = dxp_out if dxp_out is not None else torch.empty_like(xp)
            kernels.gemm(dgu, w13.view(E * twoF, H), dxp, mode=GEMM_GROUPED_M, N=H, K=twoF, b_mn=True, groups=E,
                         b_group_rows=twoF, tile_group=plan.tile_group, num_m_tiles=plan.num_m_tiles,
                         max_m_tiles=plan.max_m_tiles)
    dw2 = _weight_grad(dyp, hact, w2, H, Fdim, plan)
    dw13 = _weight_grad(dgu, xp, w13, twoF, H, plan)
    return dxp, dw13, dw2


def _local_fused() -> bool:
    """Gather and combine transfers run as kernels of their own (default) or inside the grouped GEMMs
    (``CMOE_LOCAL_FUSED=1``; measured slightly slower on one B200: the row-pull warps cost the GEMM about what the
    separate gather kernel costs)."""
    import os

    return os.environ.get("CMOE_LOCAL_FUSED", "0") != "0"


class _LocalMoEFn(torch.autograd.Function):
    """Route-sorted expert FFN on one GPU: plan -> gather -> grouped SwiGLU GEMMs -> weighted combine.

    Fused form (``CMOE_LOCAL_FUSED=1``): the first GEMM of each direction brings its own rows in (row-pull warps reading the token
    buffer through a one-entry "peer" table, so the gather overlaps the MMAs), and the last GEMM of each direction
    stores its result rows at their (token, k) slot, which turns the combine into a streaming weighted sum of K
    consecutive rows instead of an indexed gather."""

    @staticmethod
    def forward(ctx, x, gate_w32, idx32, w13, w2, capacity: int, holder: Optional[dict]):
        E = w13.shape[0]
        N, K = idx32.shape
        H = x.shape[1]
        plan = kernels.moe_plan(idx32, E, capacity=capacity)
        fused = _local_fused() and H % 8 == 0
        ctx.fused = fused
        if fused:
            x = x.contiguous()
            xp = torch.empty(plan.cap_rows, H, device=x.device, dtype=torch.bfloat16)
            ar = torch.arange(N * K, device=x.device, dtype=torch.int32)
            ident = torch.where(plan.slot_row >= 0, ar, torch.full_like(ar, -1))  # slot -> its own row, -1 if dropped
            ys = torch.empty(N * K, H, device=x.device, dtype=torch.bfloat16)
            hact, gu, _ = grouped_swiglu_forward(
                xp, w13, w2, plan, pull=dict(src_ptrs=[x.data_ptr()], slots_per_src=N * K, pull_K=K, ld_src=H),
                scatter=dict(row_slot=plan.row_slot, slots_per_rank=N * K, out_ptrs=[ys.data_ptr()], out_ld=H))
            y = torch.empty(N, H, device=x.device, dtype=torch.bfloat16)
            _ext.ext().combine_rows(ys, ident, gate_w32, y, K)
            ctx.save_for_backward(xp, hact, gu, ys, gate_w32, w13, w2, ident)
        else:
            xp = kernels.gather_rows(x, plan)
            hact, gu, yp = grouped_swiglu_forward(xp, w13, w2, plan)
            y = kernels.combine_rows(yp, plan, gate_w32)
            ctx.save_for_backward(xp, hact, gu, yp, gate_w32, w13, w2)
        ctx.plan = plan
        if holder is not None:
            holder["plan"] = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        plan = ctx.plan
        dy = dy.contiguous()
        if ctx.fused:
            xp, hact, gu, ys, gate_w32, w13, w2, ident = ctx.saved_tensors
            N, K = gate_w32.shape
            H = xp.shape[1]
            ext = _ext.ext()
            d_gate = None
            if ctx.needs_input_grad[1]:
                d_gate = torch.empty(N, K, device=dy.device, dtype=torch.float32)
                ext.combine_bwd_w(ys, ident, dy, d_gate, K)
            dyp = torch.empty(plan.cap_rows, H, device=dy.device, dtype=torch.bfloat16)
            need_dx = ctx.needs_input_grad[0]
            dxs = torch.empty(N * K, H, device=dy.device, dtype=torch.bfloat16) if need_dx else None
            _, dw13, dw2 = grouped_swiglu_backward(
                dyp, xp, hact, gu, w13, w2, plan, need_dx=need_dx,
                pull=dict(src_ptrs=[dy.data_ptr()], slots_per_src=N * K, pull_K=K, ld_src=H,
                          slot_scale=gate_w32.reshape(-1)),
                scatter=dict(row_slot=plan.row_slot, slots_per_rank=N * K, out_ptrs=[dxs.data_ptr()], out_ld=H)
                if need_dx else None)
            dx = None
            if need_dx:
                dx = torch.empty(N, H, device=dy.device, dtype=torch.bfloat16)
                ext.combine_rows(dxs, ident, None, dx, K)
            return dx, d_gate, None, dw13, dw2, None, None
        xp, hact, gu, yp, gate_w32, w13, w2 = ctx.saved_tensors
        d_gate = kernels.combine_bwd_w(yp, plan, dy) if ctx.needs_input_grad[1] else None
        dyp = kernels.gather_rows(dy, plan, slot_scale=gate_w32.reshape(-1))
        dxp, dw13, dw2 = grouped_swiglu_backward(dyp, xp, hact, gu, w13, w2, plan, need_dx=ctx.needs_input_grad[0])
        dx = kernels.combine_rows(dxp, plan, None) if dxp is not None else None
        return dx, d_gate, None, dw13, dw2, None, None


def local_moe(x: torch.Tensor, gate_w: torch.Tensor, idx: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
              capacity: int = 0, holder: Optional[dict] = None) -> torch.Tensor:
    """All experts on this rank.  ``x`` [N,H], ``gate_w`` [N,K] gate weights, ``idx`` [N,K] expert ids."""
    if on_device_path(x, w13, w2):
        return _LocalMoEFn.apply(x, gate_w.float().contiguous(), idx.to(torch.int32).contiguous(), w13, w2, capacity,
                                 holder)
    keep = None
    if capacity > 0:
        keep = ~capacity_drop_mask_reference(idx, w13.shape[0], capacity)
    return experts_reference(x, idx, gate_w, w13, w2, 0, keep)


def capacity_drop_mask_reference(idx: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """True where slot (t, k) is the (capacity+1)-th or later token of its expert *within column k*
    (first come first served in token order, each k column on its own; reference moe_layer.py:150-155)."""
    N, K = idx.shape
    drop = torch.zeros(N, K, dtype=torch.bool, device=idx.device)
    for k in range(K):
        onehot = F.one_hot(idx[:, k].long(), num_experts)
        pos = (onehot.cumsum(0) - 1).gather(1, idx[:, k : k + 1].long()).squeeze(1)
        drop[:, k] = pos >= capacity
    return drop
