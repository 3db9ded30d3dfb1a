"""Numerics of the raw sm_100a kernels against plain PyTorch fp32 restatements of the same ops.

These tests call the extension entry points directly (no autograd wrappers) so that a failure
points at one kernel.  Oracle for the router: the fp64 softmax/top-k restatement, as in the
reference's tests/test_kernels.py:41-59.
"""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DENSE, GROUPED_M, GROUPED_K = 0, 1, 2
EPI_STORE, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2


@pytest.fixture(scope="module")
def ext():
    from composed_mixture_of_experts_engine_b200.ops import _ext

    return _ext.ext()


@pytest.fixture()
def status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _gemm(ext, A, B, D, *, mode=DENSE, epi=EPI_STORE, M=0, N=0, K=0, a_mn=False, b_mn=False, groups=1,
          b_group_rows=0, split_n=0, tile_group=None, num_m_tiles=None, max_m_tiles=0, group_offsets=None,
          d_group_stride=0, accumulate=False, aux_in=None, aux_out=None, status=None):
    ext.gemm(A, B, D, mode, epi, M, N, K, a_mn, b_mn, groups, b_group_rows, split_n, tile_group, num_m_tiles,
             max_m_tiles, group_offsets, d_group_stride, accumulate, aux_in, aux_out, None, 0, 0, 0, status, 0)
    torch.cuda.synchronize()
    if status is not None:
        assert int(status.item()) == 0, f"kernel reported status {int(status.item())}"


def _rel_err(got, want):
    return float((got.float() - want.float()).norm() / (want.float().norm() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 264, 200), (1000, 1408, 2048), (4096, 4096, 4096)])
def test_gemm_dense_kmajor(ext, status, M, N, K):
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _gemm(ext, A, B, D, M=M, N=N, K=K, status=status)
    ref = A.float() @ B.float().t()
    err = _rel_err(D, ref)
    assert err < 1e-2, f"dense K-major GEMM rel err {err}"


def test_gemm_dense_fp32_accumulate(ext, status):
    torch.manual_seed(1)
    M, N, K = 256, 256, 512
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    D = torch.ones(M, N, device="cuda", dtype=torch.float32)
    _gemm(ext, A, B, D, M=M, N=N, K=K, accumulate=True, status=status)
    ref = A.float() @ B.float().t() + 1.0
    assert _rel_err(D, ref) < 1e-4


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (512, 1408, 1024)])
def test_gemm_b_nmajor(ext, status, M, N, K):
    torch.manual_seed(2)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)  # [K, N], N contiguous
    D = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _gemm(ext, A, B, D, M=M, N=N, K=K, b_mn=True, status=status)
    ref = A.float() @ B.float()
    err = _rel_err(D, ref)
    assert err < 1e-2, f"N-major B rel err {err}"


@pytest.mark.parametrize("M,N,rows", [(128, 256, [64]), (256, 512, [128, 0, 384]), (2048, 1024, [256, 128, 640, 0])])
def test_gemm_grouped_k(ext, status, M, N, rows):
    """D[g] = A[rows_g, :M]^T @ B[rows_g, :N]: the weight-gradient contraction."""
    torch.manual_seed(3)
    G = len(rows)
    offs = [0]
    for r in rows:
        offs.append(offs[-1] + r)
    R = max(offs[-1], 64)
    A = torch.randn(R, M, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(R, N, device="cuda", dtype=torch.bfloat16)
    D = torch.full((G, M, N), 7.0, device="cuda", dtype=torch.float32)
    go = torch.tensor(offs, device="cuda", dtype=torch.int32)
    _gemm(ext, A, B, D, mode=GROUPED_K, M=M, N=N, a_mn=True, b_mn=True, groups=G, group_offsets=go,
          d_group_stride=M * N, status=status)
    for g in range(G):
        ref = A[offs[g]:offs[g + 1]].float().t() @ B[offs[g]:offs[g + 1]].float()
        if rows[g] == 0:
            assert float(D[g].abs().max()) == 0.0
        else:
            err = _rel_err(D[g], ref)
            assert err < 1e-4, f"group {g} rel err {err}"


def _make_groups(counts, device="cuda"):
    """128-row padded layout for the given per-expert row counts."""
    offs, tiles = [0], []
    for e, c in enumerate(counts):
        padded = (c + 127) // 128 * 128
        tiles += [e] * (padded // 128)
        offs.append(offs[-1] + padded)
    return offs, tiles


@pytest.mark.parametrize("H,F,counts", [(128, 256, [100, 0, 300, 128]), (2048, 1024, [513, 77, 1024, 1])])
def test_grouped_swiglu_fwd_bwd(ext, status, H, F, counts):
    torch.manual_seed(4)
    E = len(counts)
    offs, tiles = _make_groups(counts)
    R = offs[-1]
    cap_tiles = len(tiles) + 3
    X = torch.zeros(cap_tiles * 128, H, device="cuda", dtype=torch.bfloat16)
    for e, c in enumerate(counts):
        X[offs[e]:offs[e] + c] = torch.randn(c, H, device="cuda", dtype=torch.bfloat16)
    W13 = (torch.randn(E, 2 * F, H, device="cuda") / math.sqrt(H)).to(torch.bfloat16)
    W2 = (torch.randn(E, H, F, device="cuda") / math.sqrt(F)).to(torch.bfloat16)
    tg = torch.full((cap_tiles,), -1, device="cuda", dtype=torch.int32)
    tg[: len(tiles)] = torch.tensor(tiles, device="cuda", dtype=torch.int32)
    nt = torch.tensor([len(tiles)], device="cuda", dtype=torch.int32)

    Hact = torch.zeros(cap_tiles * 128, F, device="cuda", dtype=torch.bfloat16)
    GU = torch.zeros(cap_tiles * 128, 2 * F, device="cuda", dtype=torch.bfloat16)
    _gemm(ext, X, W13.view(-1, H), Hact, mode=GROUPED_M, epi=EPI_SWIGLU_FWD, N=F, K=H, groups=E, b_group_rows=2 * F,
          split_n=F, tile_group=tg, num_m_tiles=nt, max_m_tiles=cap_tiles, aux_out=GU, status=status)
    Y = torch.zeros(cap_tiles * 128, H, device="cuda", dtype=torch.bfloat16)
    _gemm(ext, Hact, W2.view(-1, F), Y, mode=GROUPED_M, N=H, K=F, groups=E, b_group_rows=H, tile_group=tg,
          num_m_tiles=nt, max_m_tiles=cap_tiles, status=status)

    # fp32 restatement
    for e, c in enumerate(counts):
        if c == 0:
            continue
        x = X[offs[e]:offs[e] + c].float()
        g = x @ W13[e, :F].float().t()
        u = x @ W13[e, F:].float().t()
        h = torch.nn.functional.silu(g) * u
        y = h.to(torch.bfloat16).float() @ W2[e].float().t()
        assert _rel_err(GU[offs[e]:offs[e] + c, :F], g) < 1e-2
        assert _rel_err(GU[offs[e]:offs[e] + c, F:], u) < 1e-2
        assert _rel_err(Hact[offs[e]:offs[e] + c], h) < 1.5e-2
        assert _rel_err(Y[offs[e]:offs[e] + c], y) < 1.5e-2

    # backward pieces
    dY = torch.zeros_like(Y)
    for e, c in enumerate(counts):
        dY[offs[e]:offs[e] + c] = torch.randn(c, H, device="cuda", dtype=torch.bfloat16)
    dGU = torch.zeros_like(GU)
    _gemm(ext, dY, W2.view(-1, F), dGU, mode=GROUPED_M, epi=EPI_SWIGLU_BWD, N=F, K=H, b_mn=True, groups=E,
          b_group_rows=H, tile_group=tg, num_m_tiles=nt, max_m_tiles=cap_tiles, aux_in=GU, status=status)
    dX = torch.zeros_like(X)
    _gemm(ext, dGU, W13.view(-1, H), dX, mode=GROUPED_M, N=H, K=2 * F, b_mn=True, groups=E, b_group_rows=2 * F,
          tile_group=tg, num_m_tiles=nt, max_m_tiles=cap_tiles, status=status)
    go = torch.tensor(offs, device="cuda", dtype=torch.int32)
    dW2 = torch.zeros(E, H, F, device="cuda", dtype=torch.float32)
    _gemm(ext, dY, Hact, dW2, mode=GROUPED_K, M=H, N=F, a_mn=True, b_mn=True, groups=E, group_offsets=go,
          d_group_stride=H * F, status=status)
    dW13 = torch.zeros(E, 2 * F, H, device="cuda", dtype=torch.float32)
    _gemm(ext, dGU, X, dW13, mode=GROUPED_K, M=2 * F, N=H, a_mn=True, b_mn=True, groups=E, group_offsets=go,
          d_group_stride=2 * F * H, status=status)

    for e, c in enumerate(counts):
        if c == 0:
            assert float(dW2[e].abs().max()) == 0.0
            continue
        sl = slice(offs[e], offs[e] + c)
        x = X[sl].float().requires_grad_(True)
        w13 = W13[e].float().requires_grad_(True)
        w2 = W2[e].float().requires_grad_(True)
        g = GU[sl, :F].float()
        u = GU[sl, F:].float()
        dh = dY[sl].float() @ w2.detach()
        s = torch.sigmoid(g)
        dg = dh * u * (s * (1 + g * (1 - s)))
        du = dh * g * s
        assert _rel_err(dGU[sl, :F], dg) < 1.5e-2
        assert _rel_err(dGU[sl, F:], du) < 1.5e-2
        dgu = dGU[sl].float()
        assert _rel_err(dX[sl], dgu @ w13.detach()) < 1.5e-2
        assert _rel_err(dW2[e], dY[sl].float().t() @ Hact[sl].float()) < 1e-3
        assert _rel_err(dW13[e], dgu.t() @ X[sl].float()) < 1e-3


def _route_fp64(x, w, k):
    logits = x.double() @ w.double()
    p = torch.softmax(logits, dim=-1)
    vals, idx = torch.topk(p, k, dim=-1)
    return idx, vals / vals.sum(-1, keepdim=True), logits, p


@pytest.mark.parametrize("N,H,E,K", [(512, 256, 16, 2), (1000, 512, 64, 2), (4096, 2048, 64, 8), (300, 128, 8, 1), (2048, 1024, 128, 4)])
def test_router_fwd_bwd(ext, status, N, H, E, K):
    torch.manual_seed(5)
    x = torch.randn(N, H, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(H, E, device="cuda") / math.sqrt(H)).to(torch.bfloat16)
    logits = torch.empty(N, E, device="cuda", dtype=torch.float32)
    idx = torch.empty(N, K, device="cuda", dtype=torch.int32)
    tw = torch.empty(N, K, device="cuda", dtype=torch.float32)
    lse = torch.empty(N, device="cuda", dtype=torch.float32)
    counts = torch.empty(E, device="cuda", dtype=torch.int32)
    mean_prob = torch.empty(E, device="cuda", dtype=torch.float32)
    stats = torch.zeros(4, device="cuda", dtype=torch.float32)
    ws = torch.zeros(3 * E + 4, device="cuda", dtype=torch.int32)  # csrc/router.cuh: router_workspace_words
    for _ in range(2):  # twice: the workspace must come back clean
        ext.router_fwd(x, w, K, logits, idx, tw, lse, counts, mean_prob, stats, ws, status, 0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert int(ws.abs().sum().item()) == 0

    ridx, rw, rlogits, rp = _route_fp64(x, w, K)
    assert torch.allclose(logits.double(), rlogits, atol=2e-3, rtol=1e-3)
    # indices: exact except near-ties
    mism = (idx.long() != ridx)
    if mism.any():
        rows = mism.any(-1).nonzero().flatten()
        for r in rows.tolist()[:50]:
            got = rp[r, idx[r].long()]
            want = rp[r, ridx[r]]
            assert torch.allclose(got, want, rtol=1e-3, atol=1e-6), f"row {r}: {idx[r].tolist()} vs {ridx[r].tolist()}"
        assert mism.float().mean() < 1e-3
    ok_rows = ~mism.any(-1)
    assert torch.allclose(tw[ok_rows].double(), rw[ok_rows], atol=2e-3, rtol=2e-3)
    assert torch.allclose(tw.sum(-1), torch.ones(N, device="cuda"), atol=1e-5)
    # statistics
    bc = torch.bincount(idx.long().flatten(), minlength=E)
    assert torch.equal(counts.long(), bc)
    assert int(stats[3].item()) == N * K
    assert torch.allclose(mean_prob.double(), rp.mean(0), atol=1e-4, rtol=1e-3)
    aux_ref = E * float(((bc.double() / (N * K)) * rp.mean(0)).sum())
    assert abs(float(stats[0]) - aux_ref) < 1e-3 * max(1.0, abs(aux_ref))
    z_ref = float((torch.logsumexp(rlogits, -1) ** 2).mean())
    assert abs(float(stats[1]) - z_ref) < 2e-3 * max(1.0, abs(z_ref))
    assert abs(float(stats[2]) - float(bc.max()) / (N * K / E)) < 1e-3

    # backward: compare with autograd through the same softmax/top-k on the kernel's logits
    gw = torch.randn(N, K, device="cuda", dtype=torch.float32)
    ga = torch.tensor([0.01], device="cuda")
    gz = torch.tensor([0.001], device="cuda")
    gl = torch.empty(N, E, device="cuda", dtype=torch.float32)
    glb = torch.empty(N, E, device="cuda", dtype=torch.bfloat16)
    ext.router_bwd(logits, lse, idx, gw, counts, ga, gz, glb, gl)
    torch.cuda.synchronize()
    lg = logits.double().requires_grad_(True)
    p = torch.softmax(lg, -1)
    sel = torch.gather(p, 1, idx.long())
    wn = sel / sel.sum(-1, keepdim=True)
    f = counts.double() / (N * K)
    loss = (wn * gw.double()).sum() + 0.01 * E * (f * p.mean(0)).sum() + 0.001 * (torch.logsumexp(lg, -1) ** 2).mean()
    loss.backward()
    assert torch.allclose(gl.double(), lg.grad, atol=1e-5, rtol=1e-3), float((gl.double() - lg.grad).abs().max())
    assert _rel_err(glb, lg.grad) < 1e-2


@pytest.mark.parametrize("rows,H", [(37, 128), (512, 2048), (100, 4096), (5000, 2048), (70, 8192)])
def test_rmsnorm(ext, rows, H):
    torch.manual_seed(6)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
    ext.rmsnorm_fwd(x, w, y, rstd, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    assert _rel_err(y, ref) < 5e-3
    dy = torch.randn_like(x)
    dx = torch.empty_like(x)
    dw = torch.zeros(H, device="cuda", dtype=torch.float32)
    ext.rmsnorm_bwd(dy, x, w, rstd, dx, dw)
    ref.backward(dy.float())
    assert _rel_err(dx, xf.grad) < 5e-3
    assert _rel_err(dw, wf.grad) < 1e-3


def test_rope_roundtrip_and_reference(ext):
    torch.manual_seed(7)
    B, S, nh, hd = 2, 64, 4, 64
    t = torch.randn(B * S, nh, hd, device="cuda", dtype=torch.bfloat16)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    orig = t.clone()
    ext.rope(t, cos, sin, S, False)
    x = orig.float().view(B, S, nh, hd)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).view(B * S, nh, hd)
    assert _rel_err(t, ref) < 5e-3
    ext.rope(t, cos, sin, S, True)
    assert _rel_err(t, orig) < 1e-2


@pytest.mark.parametrize("nh,nkv", [(4, 4), (8, 2)])
def test_qkv_grad_pack_undoes_rope_and_packs(ext, nh, nkv):
    """Packing dq / dk / dv (strided [B, h, S, hd] views) into one [B, S, heads, hd] gradient with the transpose of the
    rotation applied to the q and k heads vs slicing + the fp32 restatement of the inverse rotation."""
    from composed_mixture_of_experts_engine_b200.ops import functional as OF

    torch.manual_seed(21)
    B, S, hd = 2, 96, 64
    heads = nh + 2 * nkv
    cos, sin = OF.rope_tables(S, hd, 10000.0, torch.device("cuda"))
    # sources laid out like attention gradients usually are: [B, S, h, hd] memory viewed as [B, h, S, hd]
    dq = torch.randn(B, S, nh, hd, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    dk = torch.randn(B, nkv, S, hd, device="cuda", dtype=torch.bfloat16)  # and one dense [B, h, S, hd]
    dv = torch.randn(B, S, nkv, hd, device="cuda", dtype=torch.bfloat16).permute(0, 2, 1, 3)
    out = torch.full((B, S, heads, hd), 5.0, device="cuda", dtype=torch.bfloat16)
    ext.qkv_grad_pack(dq, dk, dv, out, cos, sin)
    packed = torch.cat([dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)], dim=2).float()
    want = OF.rope_reference(packed.reshape(B * S, heads, hd), cos, -sin, S, nh + nkv).view(B, S, heads, hd)
    assert _rel_err(out, want) < 5e-3
    assert torch.equal(out[:, :, nh + nkv:], dv.permute(0, 2, 1, 3))


@pytest.mark.parametrize("n,bf16_grad", [(1000, False), (4099, True), (1 << 20, True)])
def test_adamw_matches_torch(ext, n, bf16_grad):
    torch.manual_seed(8)
    p = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        if bf16_grad:
            g = g.to(torch.bfloat16)
        ref_p.grad = g.float().clone()
        opt.step()
        ext.adamw(p, p16, m, v, g.clone(), 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, 0.0, None, False)
    assert torch.allclose(p, ref_p.detach(), atol=1e-6, rtol=1e-5)
    assert torch.equal(p16, p.to(torch.bfloat16))


def test_adamw_clip_and_sumsq(ext):
    torch.manual_seed(9)
    n = 10000
    g = torch.randn(n, device="cuda") * 5
    ss = torch.zeros(1, device="cuda")
    ext.sumsq(g, ss)
    ext.sumsq(g.to(torch.bfloat16), ss)
    want = float(g.double().pow(2).sum() + g.to(torch.bfloat16).double().pow(2).sum())
    assert abs(float(ss) - want) / want < 1e-4
    ss.zero_()
    ext.sumsq(g, ss)
    p = torch.zeros(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    gc = g.clone()
    ext.adamw(p, None, m, v, gc, 1e-3, 0.9, 0.95, 1e-8, 0.0, 1, 1.0, 1.0, ss, True)
    clip = min(1.0, 1.0 / (float(g.norm()) + 1e-6))
    assert torch.allclose(m, 0.1 * g * clip, atol=1e-6, rtol=1e-4)
    assert float(gc.abs().max()) == 0.0


@pytest.mark.parametrize("rows,V", [(64, 1024), (33, 50304)])
def test_cross_entropy(ext, rows, V):
    torch.manual_seed(10)
    logits = (torch.randn(rows, V, device="cuda") * 3).to(torch.bfloat16)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[0] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=-100, reduction="sum")
    ref.backward()
    loss = torch.zeros(1, device="cuda")
    work = logits.clone()
    ext.cross_entropy(work, tgt, loss, 1.0)
    assert abs(float(loss) - float(ref)) / abs(float(ref)) < 2e-3
    assert _rel_err(work, lf.grad) < 1e-2


@pytest.mark.parametrize("N,K,E,cap", [(1000, 2, 8, 0), (4096, 8, 64, 0), (777, 2, 16, 60), (3000, 6, 64, 0),
                                       (50000, 8, 8, 0), (20000, 4, 64, 900)])
def test_moe_plan_gather_combine(ext, N, K, E, cap):
    torch.manual_seed(11)
    H = 128
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(N)]).to(torch.int32)
    per_k = cap > 0
    cap_rows = ((N * K + E * 127) + 127) // 128 * 128
    slot_row = torch.empty(N * K, device="cuda", dtype=torch.int32)
    row_slot = torch.empty(cap_rows, device="cuda", dtype=torch.int32)
    goffs = torch.empty(E + 1, device="cuda", dtype=torch.int32)
    tg = torch.empty(cap_rows // 128, device="cuda", dtype=torch.int32)
    nt = torch.empty(1, device="cuda", dtype=torch.int32)
    kept = torch.empty(E, device="cuda", dtype=torch.int32)
    scratch = torch.empty(ext.moe_plan_scratch_words(N * K, E, K, per_k), device="cuda", dtype=torch.int32)
    ext.moe_plan(idx, K, E, 0, E, per_k, cap, slot_row, row_slot, goffs, tg, nt, kept, scratch, None)
    torch.cuda.synchronize()
    idx_c, sr, rs, go = idx.cpu().long(), slot_row.cpu(), row_slot.cpu(), goffs.cpu()
    # reference layout on the CPU
    flat = idx_c.flatten()
    want_kept = torch.zeros(E, dtype=torch.long)
    for e in range(E):
        if per_k:
            want_kept[e] = sum(min(int((idx_c[:, k] == e).sum()), cap) for k in range(K))
        else:
            want_kept[e] = int((flat == e).sum())
    assert torch.equal(kept.cpu().long(), want_kept)
    off = 0
    for e in range(E):
        assert int(go[e]) == off
        off += (int(want_kept[e]) + 127) // 128 * 128
    assert int(go[E]) == off and int(nt.item()) == off // 128
    # every kept slot sits inside its expert's segment, rows are unique, order is stable by slot
    live = sr >= 0
    assert int(live.sum()) == int(want_kept.sum())
    rows_live = sr[live].long()
    assert rows_live.unique().numel() == rows_live.numel()
    e_of_slot = flat[live]
    assert bool(((rows_live >= go[e_of_slot]) & (rows_live < go[e_of_slot] + want_kept[e_of_slot])).all())
    assert torch.equal(rs[rows_live].long(), live.nonzero().flatten())
    if not per_k:
        for e in range(0, E, max(1, E // 8)):
            slots = (flat == e).nonzero().flatten()
            assert torch.equal(sr[slots].long(), int(go[e]) + torch.arange(slots.numel()))
    else:
        for e in range(0, E, max(1, E // 4)):
            for k in range(K):
                toks = (idx_c[:, k] == e).nonzero().flatten()
                rows_k = sr[toks * K + k]
                assert bool((rows_k[:cap] >= 0).all()) and bool((rows_k[cap:] == -1).all())
    tiles = tg.cpu()[: int(nt.item())]
    for t in range(int(nt.item())):
        e = int(tiles[t])
        assert go[e] <= t * 128 < go[e + 1]

    # gather + combine against index arithmetic
    x = torch.randn(N, H, device="cuda", dtype=torch.bfloat16)
    xp = torch.full((cap_rows, H), 3.0, device="cuda", dtype=torch.bfloat16)
    ext.gather_rows(x, row_slot, K, None, xp, nt)
    n_rows = int(nt.item()) * 128
    want = torch.zeros(n_rows, H, device="cuda", dtype=torch.bfloat16)
    rsl = row_slot[:n_rows].long()
    want[rsl >= 0] = x[(rsl[rsl >= 0] // K)]
    assert torch.equal(xp[:n_rows], want)
    w = torch.rand(N, K, device="cuda")
    y = torch.empty(N, H, device="cuda", dtype=torch.bfloat16)
    ext.combine_rows(xp, slot_row, w, y, K)
    srl = slot_row.view(N, K).long()
    gathered = torch.where((srl >= 0)[..., None], xp[srl.clamp(min=0)].float(), torch.zeros((), device="cuda"))
    ref = (gathered * w[..., None]).sum(1)
    assert _rel_err(y, ref) < 5e-3
    dy = torch.randn(N, H, device="cuda", dtype=torch.bfloat16)
    dw = torch.empty(N, K, device="cuda")
    ext.combine_bwd_w(xp, slot_row, dy, dw, K)
    ref_dw = (gathered * dy.float()[:, None, :]).sum(-1)
    assert torch.allclose(dw, ref_dw, atol=1e-2, rtol=1e-2)


def test_gemm_with_fused_row_pull_matches_gather_then_gemm(ext, status):
    """The grouped GEMM that pulls its own A rows (fused dispatch) vs gather_rows followed by the plain GEMM.
    One GPU stands in for every rank: the "peer" table holds two local token buffers."""
    from composed_mixture_of_experts_engine_b200.ops import kernels
    from composed_mixture_of_experts_engine_b200.ops.kernels import EPI_SWIGLU_FWD as SWF

    torch.manual_seed(12)
    T, K, E, H, F = 1500, 4, 8, 512, 256
    xs = [torch.randn(T, H, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    x_all = torch.cat(xs)
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(2 * T)]).to(torch.int32)
    plan = kernels.moe_plan(idx, E)
    W13 = (torch.randn(E, 2 * F, H, device="cuda") / math.sqrt(H)).to(torch.bfloat16)
    scale = torch.rand(2 * T * K, device="cuda")
    for use_scale in (False, True):
        sc = scale if use_scale else None
        xp_ref = kernels.gather_rows(x_all, plan, slot_scale=sc)
        h_ref = torch.empty(plan.cap_rows, F, device="cuda", dtype=torch.bfloat16)
        gu_ref = torch.empty(plan.cap_rows, 2 * F, device="cuda", dtype=torch.bfloat16)
        kernels.gemm(xp_ref, W13.view(-1, H), h_ref, mode=GROUPED_M, epilogue=SWF, N=F, K=H, groups=E,
                     b_group_rows=2 * F, split_n=F, tile_group=plan.tile_group, num_m_tiles=plan.num_m_tiles,
                     max_m_tiles=plan.max_m_tiles, aux_out=gu_ref)
        xp = torch.full((plan.cap_rows, H), 9.0, device="cuda", dtype=torch.bfloat16)
        h = torch.empty_like(h_ref)
        gu = torch.empty_like(gu_ref)
        kernels.gemm_pull(xp, W13.view(-1, H), h, plan, epilogue=SWF, N=F, K=H, groups=E, b_group_rows=2 * F,
                          split_n=F, aux_out=gu, src_ptrs=[t.data_ptr() for t in xs], slots_per_src=T * K, pull_K=K,
                          ld_src=H, slot_scale=sc)
        torch.cuda.synchronize()
        kernels.check_status(torch.device("cuda", 0))
        n = int(plan.num_m_tiles) * 128
        assert torch.equal(xp[:n], xp_ref[:n])
        assert torch.equal(h[:n], h_ref[:n]) and torch.equal(gu[:n], gu_ref[:n])


def test_gemm_with_fused_scatter_matches_gemm_then_scatter(ext, status):
    """The grouped GEMM whose epilogue stores each result row at the home of its slot (fused combine push) vs the
    plain grouped GEMM followed by an index copy.  Two local buffers stand in for the two ranks."""
    from composed_mixture_of_experts_engine_b200.ops import kernels

    torch.manual_seed(13)
    T, K, E, H, F = 1100, 2, 4, 256, 512
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(2 * T)]).to(torch.int32)
    plan = kernels.moe_plan(idx, E)
    hact = torch.randn(plan.cap_rows, F, device="cuda", dtype=torch.bfloat16)
    W2 = (torch.randn(E, H, F, device="cuda") / math.sqrt(F)).to(torch.bfloat16)
    yp = torch.empty(plan.cap_rows, H, device="cuda", dtype=torch.bfloat16)
    kernels.gemm(hact, W2.view(-1, F), yp, mode=GROUPED_M, N=H, K=F, groups=E, b_group_rows=H,
                 tile_group=plan.tile_group, num_m_tiles=plan.num_m_tiles, max_m_tiles=plan.max_m_tiles)
    outs = [torch.full((T * K, H), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    kernels.gemm_scatter(hact, W2.view(-1, F), N=H, K=F, row_slot=plan.row_slot, slots_per_rank=T * K,
                         out_ptrs=[o.data_ptr() for o in outs], out_ld=H, plan=plan, groups=E, b_group_rows=H)
    torch.cuda.synchronize()
    kernels.check_status(torch.device("cuda", 0))
    n = int(plan.num_m_tiles) * 128
    slot = plan.row_slot[:n].long()
    live = slot >= 0
    assert int(live.sum()) == 2 * T * K  # no capacity limit: every slot has a row
    want = torch.empty(2 * T * K, H, device="cuda", dtype=torch.bfloat16)
    want[slot[live]] = yp[:n][live]
    assert torch.equal(torch.cat(outs), want)


def test_row_kernels_skip_and_report_a_slot_that_names_no_buffer(ext):
    """A corrupted row plan (a slot that points at a rank the peer table has no buffer for) must not turn into a
    stray access: the row kernels leave such rows zero, record the bad index in the status word and carry on."""
    from composed_mixture_of_experts_engine_b200.ops import kernels

    dev = torch.device("cuda", 0)
    kernels.check_status(dev)  # start from a clean word
    T, H = 256, 128
    src = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    slots = torch.arange(128, device="cuda", dtype=torch.int32)
    slots[5] = 3 * T + 7      # rank 3 of a one-entry table
    slots[9] = 40 * T + 1     # beyond the table altogether
    out = torch.full((128, H), 5.0, device="cuda", dtype=torch.bfloat16)
    tiles = torch.tensor([1], device="cuda", dtype=torch.int32)
    ext.gather_rows_peer([src.data_ptr()], T, 1, slots, None, out, tiles, H)
    torch.cuda.synchronize()
    good = [i for i in range(128) if i not in (5, 9)]
    assert torch.equal(out[good], src[good])
    assert float(out[5].abs().max()) == 0.0 and float(out[9].abs().max()) == 0.0
    with pytest.raises(kernels.KernelTimeoutError, match="outside the buffers"):
        kernels.check_status(dev)
    kernels.check_status(dev)  # the word was cleared by the failed check


def test_bounded_wait_reports_a_status_instead_of_hanging(ext):
    """A barrier whose second participant never arrives: the wait runs out after a few milliseconds, the kernel
    returns normally with status 5 (peer flag never written) and the context stays usable."""
    import time

    flags = torch.zeros(16, device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    ptrs = [flags.data_ptr(), flags.data_ptr()]  # "rank 1" is never launched, so word [1] stays 0
    t0 = time.perf_counter()
    ext.peer_barrier(ptrs, 0, 1, status, 5_000_000)  # 5 ms budget
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    assert int(status.item()) == 5 and int(flags[0]) == 1 and int(flags[1]) == 0
    # the same barrier completes at once when the other word has been written
    status.zero_()
    flags[1] = 2
    ext.peer_barrier(ptrs, 0, 2, status, 5_000_000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0  # the context is alive
