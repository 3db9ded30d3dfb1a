"""CPU restatement (fp64) of the tile schedules of csrc/attention.cu, checked against plain causal attention.

The forward keeps, per query row, a running maximum in the base-2 domain, a running sum and an output row that is
rescaled by ``alpha`` of the *previous* tile when that tile's partial product is added (the partial product of tile
i is read back while tile i+1 is in its softmax).  The backward walks the query tiles at or below a key tile's
diagonal and forms P from the saved log-sum-exp, dS = P (dP - delta) scale, and the three gradient products.
These tests pin that arithmetic independently of the GPU; the kernels themselves are tested in
tests/test_gpu_attention.py.
"""

from __future__ import annotations

import math

import pytest
import torch

BLK = 128


def _reference(q, k, v):
    S, hd = q.shape
    scores = (q @ k.T) / math.sqrt(hd)
    mask = torch.ones(S, S, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(scores, -1) @ v, torch.logsumexp(scores, -1)


def _forward_tiled(q, k, v):
    S, hd = q.shape
    T = S // BLK
    sl2 = math.log2(math.e) / math.sqrt(hd)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, dtype=q.dtype)
    rows = torch.arange(BLK)
    for qt in range(T):
        Q = q[qt * BLK:(qt + 1) * BLK]
        O = torch.zeros(BLK, hd, dtype=q.dtype)
        m = torch.full((BLK,), -float("inf"), dtype=q.dtype)
        l = torch.zeros(BLK, dtype=q.dtype)
        alpha_saved = torch.zeros(BLK, dtype=q.dtype)
        pv = [None, None]
        for i in range(qt + 1):
            st = i & 1
            s = Q @ k[i * BLK:(i + 1) * BLK].T
            limit = rows if i == qt else torch.full((BLK,), BLK)
            valid = torch.arange(BLK)[None, :] <= limit[:, None]
            mx = s.masked_fill(~valid, -float("inf")).max(-1).values
            m_new = torch.maximum(m, mx * sl2)
            alpha = torch.exp2(m - m_new)
            p = torch.exp2(s * sl2 - m_new[:, None]) * valid
            l = l * alpha + p.sum(-1)
            m = m_new
            pv[st] = p @ v[i * BLK:(i + 1) * BLK]
            if i > 0:
                O = O * alpha_saved[:, None] + pv[st ^ 1]
            alpha_saved = alpha
        O = O * alpha_saved[:, None] + pv[qt & 1]
        out[qt * BLK:(qt + 1) * BLK] = O / l[:, None]
        lse[qt * BLK:(qt + 1) * BLK] = (m + torch.log2(l)) * math.log(2)
    return out, lse


def _forward_lazy_rescale(q, k, v, threshold=8.0):
    """The two-query-tile kernel (csrc/attention_fwd2.cu): O accumulates across key tiles and is rescaled only when
    the row maximum has grown by more than ``threshold`` (base 2) since the value the probabilities are taken
    against was last moved; in between that value is stale and the probabilities exceed 1 by at most 2^threshold."""
    S, hd = q.shape
    T = S // BLK
    sl2 = math.log2(math.e) / math.sqrt(hd)
    out = torch.zeros_like(q)
    lse = torch.zeros(S, dtype=q.dtype)
    rows = torch.arange(BLK)
    rescales = 0
    for qt in range(T):
        Q = q[qt * BLK:(qt + 1) * BLK]
        O = torch.zeros(BLK, hd, dtype=q.dtype)
        m_used = torch.full((BLK,), -float("inf"), dtype=q.dtype)
        l = torch.zeros(BLK, dtype=q.dtype)
        for i in range(qt + 1):
            s = Q @ k[i * BLK:(i + 1) * BLK].T
            limit = rows if i == qt else torch.full((BLK,), BLK)
            valid = torch.arange(BLK)[None, :] <= limit[:, None]
            mx = s.masked_fill(~valid, -float("inf")).max(-1).values
            m_new = torch.maximum(m_used, mx * sl2)
            grow = (m_new - m_used) > threshold
            alpha = torch.where(grow, torch.exp2(m_used - m_new), torch.ones_like(m_new))
            m_used = torch.where(grow, m_new, m_used)
            p = torch.exp2(s * sl2 - m_used[:, None]) * valid
            assert float(p.max()) <= 2.0 ** threshold * (1 + 1e-9)
            l = l * alpha + p.sum(-1)
            if i > 0:
                rescales += int(grow.any())
                O = O * alpha[:, None]
            O = O + p @ v[i * BLK:(i + 1) * BLK]
        out[qt * BLK:(qt + 1) * BLK] = O / l[:, None]
        lse[qt * BLK:(qt + 1) * BLK] = (m_used + torch.log2(l)) * math.log(2)
    return out, lse, rescales


def _backward_tiled(q, k, v, out, lse, go):
    S, hd = q.shape
    T = S // BLK
    sc = 1 / math.sqrt(hd)
    sl2 = sc * math.log2(math.e)
    delta = (go * out).sum(-1)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    rows = torch.arange(BLK)
    for kt in range(T):
        K, V = k[kt * BLK:(kt + 1) * BLK], v[kt * BLK:(kt + 1) * BLK]
        for qt in range(kt, T):
            sl = slice(qt * BLK, (qt + 1) * BLK)
            s, dp = q[sl] @ K.T, go[sl] @ V.T
            limit = rows if qt == kt else torch.full((BLK,), BLK)
            valid = torch.arange(BLK)[None, :] <= limit[:, None]
            p = torch.exp2(s * sl2 - (lse[sl] * math.log2(math.e))[:, None]) * valid
            ds = p * (dp - delta[sl][:, None]) * sc
            dv[kt * BLK:(kt + 1) * BLK] += p.T @ go[sl]
            dk[kt * BLK:(kt + 1) * BLK] += ds.T @ q[sl]
            dq[sl] += ds @ K
    return dq, dk, dv


@pytest.mark.parametrize("S,hd", [(128, 64), (384, 64), (512, 128)])
def test_tile_schedules_match_plain_causal_attention(S, hd):
    torch.manual_seed(0)
    q, k, v, go = (torch.randn(S, hd, dtype=torch.float64) for _ in range(4))
    ref, lse_ref = _reference(q, k, v)
    out, lse = _forward_tiled(q, k, v)
    assert (out - ref).abs().max() < 1e-12 and (lse - lse_ref).abs().max() < 1e-12

    qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
    _reference(qa, ka, va)[0].backward(go)
    dq, dk, dv = _backward_tiled(q, k, v, out, lse, go)
    for got, want in ((dq, qa.grad), (dk, ka.grad), (dv, va.grad)):
        assert (got - want).abs().max() < 1e-11


def test_lazy_rescale_schedule_is_exact_and_rescales_rarely():
    torch.manual_seed(1)
    S, hd = 1024, 128
    q, k, v = (torch.randn(S, hd, dtype=torch.float64) for _ in range(3))
    ref, lse_ref = _reference(q, k, v)
    out, lse, rescales = _forward_lazy_rescale(q, k, v)
    assert (out - ref).abs().max() < 1e-12 and (lse - lse_ref).abs().max() < 1e-12
    tiles_after_first = sum(qt for qt in range(S // BLK))
    assert rescales < tiles_after_first // 2



class _FakeExt:
    """PyTorch stand-in for the extension's attention entry points (same argument lists), so that the autograd glue
    around them can be checked without a GPU."""

    @staticmethod
    def _split(qkv, nh, nkv):
        return qkv[:, :, :nh], qkv[:, :, nh: nh + nkv], qkv[:, :, nh + nkv:]

    def attention_fwd(self, qkv, nh, nkv, out, lse, status, timeout_ns):
        q, k, v = self._split(qkv.double(), nh, nkv)
        S, hd = q.shape[1], q.shape[3]
        kk = k.repeat_interleave(nh // nkv, 2)
        vv = v.repeat_interleave(nh // nkv, 2)
        scores = torch.einsum("bqhd,bkhd->bhqk", q, kk) / math.sqrt(hd)
        mask = torch.ones(S, S, dtype=torch.bool).tril()
        scores = scores.masked_fill(~mask, float("-inf"))
        out.copy_(torch.einsum("bhqk,bkhd->bqhd", torch.softmax(scores, -1), vv).to(out.dtype))
        lse.copy_(torch.logsumexp(scores, -1).to(lse.dtype))

    def attention_bwd(self, qkv, nh, nkv, out, dout, lse, delta, dq, dk, dv, status, timeout_ns):
        with torch.enable_grad():  # called from inside an autograd backward, where recording is off
            x = qkv.double().requires_grad_()
            q, k, v = self._split(x, nh, nkv)
            S, hd = q.shape[1], q.shape[3]
            scores = torch.einsum("bqhd,bkhd->bhqk", q, k.repeat_interleave(nh // nkv, 2)) / math.sqrt(hd)
            scores = scores.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
            o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(scores, -1), v.repeat_interleave(nh // nkv, 2))
            (g,) = torch.autograd.grad(o, x, dout.double())
        gq, gk, gv = self._split(g, nh, nkv)
        assert float(dq.abs().max()) == 0.0  # the kernel accumulates into dq: the caller must hand in zeros
        dq.add_(gq.to(dq.dtype))
        dk.copy_(gk.to(dk.dtype))
        dv.copy_(gv.to(dv.dtype))


def test_packed_attention_autograd_glue_with_a_stand_in_extension(monkeypatch):
    """``attention_sm100._PackedAttentionFn`` (allocation of out / lse / dq / dk / dv, zeroed dq, packing of the
    three gradients along the head axis) against plain autograd, with the kernels replaced by PyTorch."""
    from composed_mixture_of_experts_engine_b200.ops import _ext, attention_sm100 as A
    from composed_mixture_of_experts_engine_b200.ops import kernels
    from composed_mixture_of_experts_engine_b200.ops.attention import attention_reference

    monkeypatch.setattr(_ext, "ext", lambda: _FakeExt())
    monkeypatch.setattr(kernels, "status_word", lambda device: torch.zeros(1, dtype=torch.int32))
    torch.manual_seed(0)
    B, S, nh, nkv, hd = 2, 128, 4, 2, 64
    qkv = torch.randn(B, S, nh + 2 * nkv, hd, dtype=torch.bfloat16).float().requires_grad_()
    go = torch.randn(B, S, nh, hd)

    x = qkv.detach().to(torch.bfloat16).requires_grad_()
    out = A.packed_causal_attention(x, nh, nkv)
    out.backward(go.to(torch.bfloat16))

    ref = attention_reference(qkv[:, :, :nh], qkv[:, :, nh: nh + nkv], qkv[:, :, nh + nkv:])
    ref.backward(go)
    assert out.shape == (B, S, nh, hd) and x.grad.shape == qkv.shape
    assert (out.float() - ref).abs().max() < 3e-2
    assert (x.grad.float() - qkv.grad).norm() / qkv.grad.norm() < 2e-2


# ---- shared-memory operand layout ------------------------------------------------------------------------------
def _swizzle128(byte_offset: int) -> int:
    """128-byte swizzle of a 1024-byte-aligned block: bits 4-6 of the offset are XORed with bits 7-9."""
    return byte_offset ^ (((byte_offset >> 7) & 7) << 4)


def _store_swizzled(mat: dict, r: int, col: int, value) -> None:
    """Where ``store_swizzled_32`` of csrc/attention.cu puts element (r, col) of a [128 x 128] bf16 matrix: two
    blocks of [128 rows x 64 columns], 16-byte piece j of a row at piece j ^ (r % 8)."""
    block, c = divmod(col, 64)
    piece, within = divmod(c, 8)
    mat[block * 128 * 128 + r * 128 + ((piece ^ (r & 7)) << 4) + within * 2] = value


def test_probability_tile_serves_as_k_major_and_as_mn_major_operand():
    """The P / dS tile is written once and read twice by the tensor cores: as a K-major A operand (rows = queries,
    contraction over keys: P V, dS K) and as an MN-major A operand (M = keys, contraction over queries: P^T dO,
    dS^T Q).  Both canonical 128-byte-swizzle layouts must address the byte the store put there: K-major rows are
    128 bytes apart with eight-row groups 1024 bytes apart; MN-major k-rows are 128 bytes apart, 64-element M
    chunks one block (16 KiB) apart."""
    mem = {}
    for r in range(128):
        for c in range(128):
            _store_swizzled(mem, r, c, (r, c))
    block_bytes = 128 * 128
    for r in range(0, 128, 7):
        for c in range(0, 128, 5):
            # K-major: element (m = r, k = c) of the 64-wide K block c // 64
            off = (c // 64) * block_bytes + _swizzle128((r // 8) * 1024 + (r % 8) * 128 + (c % 64) * 2)
            assert mem[off] == (r, c)
            # MN-major: element (m = c, k = r): chunk c // 64 at LBO = one block, k-row r at 128 bytes
            off = (c // 64) * block_bytes + _swizzle128((r // 8) * 1024 + (r % 8) * 128 + (c % 64) * 2)
            assert mem[off] == (r, c)
    # every byte pair written exactly once
    assert len(mem) == 128 * 128
