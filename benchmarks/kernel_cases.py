"""Single-kernel cases for timing and for profiler captures.

    python benchmarks/kernel_cases.py <case> [--iters N] [--small]

Each case builds its inputs (larger than the 126 MB L2, a few GB at most), warms up, then times ``iters``
launches with CUDA events (an L2-sized buffer is overwritten between launches) and prints one JSON line with the
achieved bandwidth / throughput and the fraction of the measured peaks (MEASURED_PEAKS.json).  The same command
line under ``ncu -k regex:<kernel> -c 1`` captures one launch of the case.

Cases: adamw, rmsnorm, router / router_bwd (config-2 shape: T16384 d4096 E64 top2), gemm_dense, dense_shapes,
grouped_fwd1, grouped_fwd1_pull (fused dispatch through a local one-entry peer table), grouped_fwd2,
grouped_dgrad, grouped_wgrad, gather, combine.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from composed_mixture_of_experts_engine_b200.ops import _ext, kernels  # noqa: E402
from composed_mixture_of_experts_engine_b200.ops.kernels import (EPI_SWIGLU_BWD, EPI_SWIGLU_FWD, GEMM_GROUPED_K,  # noqa: E402
                                                                 GEMM_GROUPED_M)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def time_launches(fn, iters: int, warm: int = 3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def uniform_plan(rows: int, experts: int):
    tiles = rows // 128
    tg = (torch.arange(tiles, device="cuda", dtype=torch.int32) // (tiles // experts)).contiguous()
    nt = torch.tensor([tiles], device="cuda", dtype=torch.int32)
    go = (torch.arange(experts + 1, device="cuda", dtype=torch.int32) * (rows // experts)).contiguous()
    return tg, nt, go, tiles


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--small", action="store_true", help="quarter-size inputs (for multi-pass profiler captures)")
    ap.add_argument("--rows", type=int, default=65536, help="expert-sorted rows of the grouped cases")
    ap.add_argument("--experts", type=int, default=64, help="experts of the grouped cases")
    ap.add_argument("--hidden", type=int, default=2048, help="model width of the grouped cases")
    ap.add_argument("--ffn", type=int, default=1024, help="FFN width per expert of the grouped cases")
    ap.add_argument("--router-hidden", type=int, default=4096, help="model width of the router cases")
    ap.add_argument("--topk", type=int, default=2, help="experts per token of the router cases")
    args = ap.parse_args()
    ext = _ext.ext()
    hbm, tflops_peak, how = peaks()
    dev = "cuda"
    bf = torch.bfloat16
    out = {"case": args.case, "peaks": how}
    shrink = 4 if args.small else 1

    if args.case == "adamw":
        n = (1 << 28) // shrink
        p, m, v = (torch.randn(n, device=dev) for _ in range(3))
        g = torch.randn(n, device=dev)
        p16 = torch.empty(n, device=dev, dtype=bf)
        ms = time_launches(lambda: ext.adamw(p, p16, m, v, g, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, 0.0, None, True),
                           args.iters)
        nbytes = n * (8 + 8 + 8 + 8 + 2)
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac_of_hbm=nbytes / ms / 1e6 / hbm, elements=n)
    elif args.case == "hbm":
        # what the memory system gives a pure write, a pure read and a copy of 1 GiB (ATen kernels: reference rates
        # for the row kernels, whose traffic is mostly one-directional)
        n = 1 << 29
        x = torch.empty(n, device=dev, dtype=bf)
        y = torch.empty(n, device=dev, dtype=bf)
        w_ms = time_launches(lambda: x.fill_(1.0), args.iters)
        r_ms = time_launches(lambda: x.sum(dtype=torch.float32), args.iters)
        c_ms = time_launches(lambda: y.copy_(x), args.iters)
        gb = n * 2 / 1e6
        out.update(write_gbs=gb / w_ms, read_gbs=gb / r_ms, copy_gbs=2 * gb / c_ms)
    elif args.case == "rmsnorm":
        rows, H = 32768 // shrink, 2048
        x = torch.randn(rows, H, device=dev, dtype=bf)
        w = torch.ones(H, device=dev, dtype=bf)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        rstd = torch.empty(rows, device=dev)
        dw = torch.zeros(H, device=dev)
        f = time_launches(lambda: ext.rmsnorm_fwd(x, w, y, rstd, 1e-5), args.iters)
        b = time_launches(lambda: ext.rmsnorm_bwd(y, x, w, rstd, dx, dw), args.iters)
        nb = rows * H * 2
        out.update(fwd_ms=f, fwd_gbs=2 * nb / f / 1e6, fwd_frac=2 * nb / f / 1e6 / hbm, bwd_ms=b,
                   bwd_gbs=3 * nb / b / 1e6, bwd_frac=3 * nb / b / 1e6 / hbm)
    elif args.case == "router":
        N, H, E, K = 16384 // (2 if args.small else 1), args.router_hidden, 64, args.topk
        x = torch.randn(N, H, device=dev, dtype=bf)
        w = (torch.randn(H, E, device=dev) * 0.02).to(bf)
        from composed_mixture_of_experts_engine_b200.ops.moe_router import fused_router_forward

        ms = time_launches(lambda: fused_router_forward(x, w, K), max(args.iters, 20))
        nbytes = N * H * 2 + H * E * 2 + N * E * 4 + N * K * 8 + N * 4
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac_of_hbm=nbytes / ms / 1e6 / hbm, tokens_per_s=N / ms * 1e3)
    elif args.case == "router_bwd":
        # analytic d(logits) kernel + the two tcgen05 GEMMs of the router backward (config-2 shape by default)
        N, H, E, K = 16384 // (2 if args.small else 1), args.router_hidden, 64, args.topk
        x = torch.randn(N, H, device=dev, dtype=bf)
        w = (torch.randn(H, E, device=dev) * 0.02).to(bf)
        from composed_mixture_of_experts_engine_b200.ops.moe_router import fused_router_forward

        o = fused_router_forward(x, w, K)
        gw = torch.randn(N, K, device=dev)
        ga = torch.tensor([0.01], device=dev)
        gz = torch.tensor([0.001], device=dev)
        gl16 = torch.empty(N, E, device=dev, dtype=bf)

        def bwd():
            ext.router_bwd(o.logits, o.lse, o.idx32, gw, o.counts, ga, gz, gl16, None)
            kernels.linear_nt(gl16, w)      # grad_tokens = gl @ gate_w^T
            kernels.linear_tn(x, gl16)      # grad_gate_w = tokens^T @ gl

        ms = time_launches(bwd, max(args.iters, 20))
        only = time_launches(lambda: ext.router_bwd(o.logits, o.lse, o.idx32, gw, o.counts, ga, gz, gl16, None),
                             max(args.iters, 20))
        nbytes = N * E * 4 + N * E * 2 + 2 * N * H * 2 + H * E * 4  # logits in, gl out; tokens in, grad_tokens out
        out.update(ms=ms, dlogits_kernel_ms=only, gbs=nbytes / ms / 1e6, frac_of_hbm=nbytes / ms / 1e6 / hbm)
    elif args.case == "gemm_dense":
        M = N = K = 8192 // (2 if args.small else 1)
        A = torch.randn(M, K, device=dev, dtype=bf)
        B = torch.randn(N, K, device=dev, dtype=bf)
        D = torch.empty(M, N, device=dev, dtype=bf)
        ms = time_launches(lambda: kernels.gemm(A, B, D, M=M, N=N, K=K), args.iters)
        lib = time_launches(lambda: torch.matmul(A, B.t(), out=D), args.iters)
        fl = 2 * M * N * K
        out.update(ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tflops_peak, cublas_ms=lib,
                   cublas_tflops=fl / lib / 1e9)
    elif args.case == "dense_shapes":
        # the projections and the LM head of the headline model: forward, input gradient, weight gradient
        # (rows, in features, out features); each against torch.matmul (cuBLAS) on the same operands
        rows_out = []
        for (M, K, N) in ((16384, 2048, 6144), (16384, 2048, 2048), (4096, 2048, 50304)):
            x = torch.randn(M, K, device=dev, dtype=bf)
            w = (torch.randn(N, K, device=dev) * 0.02).to(bf)
            dy = torch.randn(M, N, device=dev, dtype=bf)
            y = torch.empty(M, N, device=dev, dtype=bf)
            dx = torch.empty(M, K, device=dev, dtype=bf)
            dw = torch.zeros(N, K, device=dev, dtype=torch.float32)
            dw16 = torch.empty(N, K, device=dev, dtype=bf)
            fl = 2 * M * N * K
            for name, own, lib in (
                    ("fwd", lambda: kernels.linear_nt(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
                    ("dgrad", lambda: kernels.linear_nn(dy, w, out=dx), lambda: torch.matmul(dy, w, out=dx)),
                    ("wgrad", lambda: kernels.linear_tn_acc(dy, x, dw), lambda: torch.matmul(dy.t(), x, out=dw16))):
                a, b = time_launches(own, args.iters), time_launches(lib, args.iters)
                rows_out.append({"shape": [M, K, N], "op": name, "ms": round(a, 4), "tflops": round(fl / a / 1e9, 1),
                                 "cublas_ms": round(b, 4), "cublas_tflops": round(fl / b / 1e9, 1),
                                 "of_cublas": round(b / a, 3), "frac_of_peak": round(fl / a / 1e9 / tflops_peak, 3)})
            del x, w, dy, y, dx, dw, dw16
        out.update(cases=rows_out)
    elif args.case.startswith("grouped_") or args.case in ("gather", "combine"):
        E, H, F = args.experts, args.hidden, args.ffn
        R = args.rows // shrink
        tg, nt, go, tiles = uniform_plan(R, E)
        X = torch.randn(R, H, device=dev, dtype=bf)
        W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.02).to(bf)
        W2 = (torch.randn(E, H, F, device=dev) * 0.02).to(bf)
        Hact = torch.randn(R, F, device=dev, dtype=bf)
        GU = torch.randn(R, 2 * F, device=dev, dtype=bf)
        Y = torch.randn(R, H, device=dev, dtype=bf)
        common = dict(groups=E, tile_group=tg, num_m_tiles=nt, max_m_tiles=tiles)
        if args.case == "grouped_fwd1":
            fn = lambda: kernels.gemm(X, W13.view(-1, H), Hact, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_FWD, N=F, K=H,
                                      b_group_rows=2 * F, split_n=F, aux_out=GU, **common)
            fl = 2 * R * 2 * F * H
        elif args.case == "grouped_fwd1_pull":
            # the same GEMM with the fused dispatch: four extra warps per CTA fill X from a token buffer through a
            # one-entry "peer" table that points at this GPU's own memory (what the pull warps cost the tensor pipe)
            Tn, Kk = R // 8, 8
            idx = torch.stack([torch.randperm(E, device=dev)[:Kk] for _ in range(Tn)]).to(torch.int32)
            plan = kernels.moe_plan(idx, E)
            tok = torch.randn(Tn, H, device=dev, dtype=bf)
            Xp = torch.empty(plan.cap_rows, H, device=dev, dtype=bf)
            Hp = torch.empty(plan.cap_rows, F, device=dev, dtype=bf)
            GUp = torch.empty(plan.cap_rows, 2 * F, device=dev, dtype=bf)
            fn = lambda st=None: kernels.gemm_pull(Xp, W13.view(-1, H), Hp, plan, epilogue=EPI_SWIGLU_FWD, N=F, K=H,
                                                   groups=E, b_group_rows=2 * F, split_n=F, aux_out=GUp,
                                                   src_ptrs=[tok.data_ptr()], slots_per_src=Tn * Kk, pull_K=Kk,
                                                   ld_src=H, stamps=st)
            fl = 2 * R * 2 * F * H
            # device timeline of one launch: first / last row pulled against first / last MMA
            st = kernels.new_pull_stamps(torch.device("cuda", 0))
            fn()
            fn(st)
            torch.cuda.synchronize()
            p0, p1, m0, m1 = (int(v) for v in st.tolist())
            out.update(timeline_us={"pull_first_to_last": (p1 - p0) / 1e3, "mma_first_to_last": (m1 - m0) / 1e3,
                                    "first_mma_after_first_pull": (m0 - p0) / 1e3})
        elif args.case == "grouped_fwd2":
            fn = lambda: kernels.gemm(Hact, W2.view(-1, F), Y, mode=GEMM_GROUPED_M, N=H, K=F, b_group_rows=H, **common)
            fl = 2 * R * F * H
        elif args.case == "grouped_dgrad":
            dGU = torch.empty_like(GU)
            fn = lambda: kernels.gemm(Y, W2.view(-1, F), dGU, mode=GEMM_GROUPED_M, epilogue=EPI_SWIGLU_BWD, N=F, K=H,
                                      b_mn=True, b_group_rows=H, aux_in=GU, **common)
            fl = 2 * R * F * H
        elif args.case in ("grouped_wgrad", "grouped_wgrad_store", "grouped_wgrad_bf16"):
            # fp32 accumulate (what training runs), fp32 overwrite, bf16 overwrite: the last two bound the main loop
            dW13 = torch.zeros(E, 2 * F, H, device=dev, dtype=bf if args.case.endswith("bf16") else torch.float32)
            acc = args.case == "grouped_wgrad"
            fn = lambda: kernels.gemm(GU, X, dW13, mode=GEMM_GROUPED_K, M=2 * F, N=H, a_mn=True, b_mn=True, groups=E,
                                      group_offsets=go, d_group_stride=2 * F * H, accumulate=acc)
            fl = 2 * R * 2 * F * H
        elif args.case == "grouped_dx":
            dX = torch.empty_like(X)
            fn = lambda: kernels.gemm(GU, W13.view(-1, H), dX, mode=GEMM_GROUPED_M, N=H, K=2 * F, b_mn=True,
                                      b_group_rows=2 * F, **common)
            fl = 2 * R * 2 * F * H
        else:
            N, K = R // 8, 8
            idx = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(N)]).to(torch.int32)
            plan = kernels.moe_plan(idx, E)
            src = torch.randn(N, H, device=dev, dtype=bf)
            rows = torch.randn(plan.cap_rows, H, device=dev, dtype=bf)
            wts = torch.rand(N, K, device=dev)
            if args.case == "gather":
                fn = lambda: kernels.gather_rows(src, plan, out=rows)
            else:
                yv = torch.empty(N, H, device=dev, dtype=bf)
                fn = lambda: kernels.combine_rows(rows, plan, wts, out=yv)
            ms = time_launches(fn, args.iters)
            nbytes = (N * K + N) * H * 2
            out.update(ms=ms, gbs=nbytes / ms / 1e6, frac_of_hbm=nbytes / ms / 1e6 / hbm)
            print(json.dumps(out))
            return
        ms = time_launches(fn, args.iters)
        out.update(ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tflops_peak, rows=R)
    else:
        raise SystemExit(f"unknown case {args.case}")
    kernels.check_status(torch.device("cuda", 0))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
