#!/usr/bin/env python
"""Causal attention micro-benchmark: the hand-written tcgen05 kernels (csrc/attention.cu) against the library
attention (cuDNN through ``scaled_dot_product_attention``) on one GPU.

    python benchmarks/attention_bench.py                      # B 4, S 4096, 16 heads, hd 128, CUDA-event timings
    python benchmarks/attention_bench.py --once --batch 2     # one warm-up + one launch of each kernel (for ncu -k)

Timing: warm-up launches, then ``--iters`` launches between two CUDA events on the launching stream; inputs are
larger than L2 at the default shape.  Prints one JSON line.  The reference has no attention operator
(pkg/models/moe.py:148-186), so there is no reference arm.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from composed_mixture_of_experts_engine_b200.ops import _ext, kernels  # noqa: E402


def _time(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--once", action="store_true", help="one warm-up and one launch per kernel, no library arm")
    a = ap.parse_args()
    B, S, nh, nkv, hd = a.batch, a.seq, a.heads, a.kv_heads, a.head_dim
    dev = torch.device("cuda:0")
    m = _ext.ext()
    st = kernels.status_word(dev)
    torch.manual_seed(0)
    qkv = torch.randn(B, S, nh + 2 * nkv, hd, device=dev).to(torch.bfloat16)
    go = torch.randn(B, S, nh, hd, device=dev).to(torch.bfloat16)
    out = torch.empty(B, S, nh, hd, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, nh, S, device=dev)
    dq = torch.zeros(B, S, nh, hd, device=dev)
    dk = torch.empty(B, S, nkv, hd, device=dev, dtype=torch.bfloat16)
    dv = torch.empty_like(dk)
    delta = torch.empty(B, nh, S, device=dev)

    def fwd():
        m.attention_fwd(qkv, nh, nkv, out, lse, st, 0)

    def bwd():
        m.attention_bwd(qkv, nh, nkv, out, go, lse, delta, dq, dk, dv, st, 0)

    if a.once:
        for _ in range(2):
            fwd()
            bwd()
        torch.cuda.synchronize()
        kernels.check_status(dev)
        print(json.dumps({"once": True, "shape": [B, S, nh, nkv, hd]}))
        return

    flops_f = 4.0 * B * nh * S * S * hd / 2
    res = {"shape": {"B": B, "S": S, "nh": nh, "nkv": nkv, "hd": hd}, "iters": a.iters, "warmup": a.warmup}
    ms = _time(fwd, a.warmup, a.iters)
    res["fwd_ms"], res["fwd_tflops"] = ms, flops_f / ms / 1e9
    ms = _time(bwd, a.warmup, a.iters)
    res["bwd_ms"], res["bwd_tflops"] = ms, 2.5 * flops_f / ms / 1e9
    kernels.check_status(dev)

    q = qkv[:, :, :nh].permute(0, 2, 1, 3).detach().requires_grad_()
    k = qkv[:, :, nh: nh + nkv].permute(0, 2, 1, 3).detach().requires_grad_()
    v = qkv[:, :, nh + nkv:].permute(0, 2, 1, 3).detach().requires_grad_()
    kk, vv = (k, v) if nkv == nh else (k.repeat_interleave(nh // nkv, 1), v.repeat_interleave(nh // nkv, 1))
    res["library_fwd_ms"] = _time(lambda: F.scaled_dot_product_attention(q, kk, vv, is_causal=True), a.warmup, a.iters)
    o = F.scaled_dot_product_attention(q, kk, vv, is_causal=True)
    g = go.permute(0, 2, 1, 3)
    res["library_bwd_ms"] = _time(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), a.warmup, a.iters)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
