"""Micro-benchmark suite: router forward / forward+backward, MoE layer vs one dense SwiGLU FFN, token conservation.

    python benchmarks/run_benchmark.py [--cuda] [--json out.json] [--csv out.csv] [--dtype bf16|fp32]

Same workloads and output fields as the reference's benchmarks/run_benchmark.py (its four router shapes
(N,H,E,K) = (512,256,16,2) (1024,512,32,2) (2048,1024,64,2) (4096,2048,64,4), its three layer shapes, the 100-seed
conservation sweep that CI gates on), plus the single-GPU router shape of the benchmark spec
(T=16384, d=4096, E=64, top-2, bf16).  Differences: GPU timings are CUDA-event timings of the device work (3 warm-up
+ 20 timed iterations, an L2-sized buffer is overwritten between iterations) instead of host wall clock, and the
GPU suite defaults to bf16 inputs, the dtype the fused sm_100a kernel consumes (``--dtype fp32`` runs the
PyTorch fp64 path on the GPU, as the reference's fp32 inputs did through Triton).
"""

from __future__ import annotations

import argparse
import csv
import json
import sys
import time
from pathlib import Path

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from composed_mixture_of_experts_engine_b200.ops.moe_router import moe_topk_route  # noqa: E402
from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer  # noqa: E402

ROUTER_CONFIGS = [(512, 256, 16, 2), (1024, 512, 32, 2), (2048, 1024, 64, 2), (4096, 2048, 64, 4)]
SPEC_ROUTER_CONFIG = (16384, 4096, 64, 2)
LAYER_CONFIGS = [(2, 16, 128, 256, 8, 2), (2, 32, 256, 512, 16, 2), (4, 16, 512, 1024, 32, 2)]
WARMUP, ITERS = 3, 20


def _time_fn(fn, device: str):
    """Median milliseconds over ITERS runs after WARMUP runs."""
    times = []
    if device == "cuda":
        flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
        for _ in range(WARMUP):
            fn()
        for _ in range(ITERS):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    else:
        for _ in range(WARMUP):
            fn()
        for _ in range(ITERS):
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    times.sort()
    return times[len(times) // 2]


def bench_router_forward(N, H, E, K, device, dtype):
    x = torch.randn(N, H, device=device, dtype=dtype)
    w = (torch.randn(H, E, device=device) / H**0.5).to(dtype)
    with torch.no_grad():
        ms = _time_fn(lambda: moe_topk_route(x, w, K), device)
    return {"bench": "router_forward", "N": N, "H": H, "E": E, "K": K, "ms": ms, "tokens_per_sec": N / ms * 1e3}


def bench_router_fwd_bwd(N, H, E, K, device, dtype):
    x = torch.randn(N, H, device=device, dtype=dtype, requires_grad=True)
    w = (torch.randn(H, E, device=device) / H**0.5).to(dtype).requires_grad_(True)
    gw = torch.randn(N, K, device=device, dtype=dtype)

    def step():
        x.grad = w.grad = None
        _, wt = moe_topk_route(x, w, K)
        (wt * gw).sum().backward()

    ms = _time_fn(step, device)
    return {"bench": "router_fwd_bwd", "N": N, "H": H, "E": E, "K": K, "ms": ms, "tokens_per_sec": N / ms * 1e3}


_layer_topology = None  # the reference's layer needs an explicit (degenerate, single-rank) topology


def bench_moe_layer(B, S, H, Fd, E, K, device, dtype):
    kw = {"topology": _layer_topology(device)} if _layer_topology is not None else {}
    layer = DistributedMoELayer(H, Fd, E, K, dtype=dtype, **kw).to(device)
    x = torch.randn(B, S, H, device=device, dtype=dtype)
    with torch.no_grad():
        ms = _time_fn(lambda: layer(x), device)
    return {"bench": "moe_layer_forward", "B": B, "S": S, "H": H, "F": Fd, "E": E, "K": K, "ms": ms}


def bench_dense_baseline(B, S, H, Fd, device, dtype):
    wg, wu = torch.randn(Fd, H, device=device, dtype=dtype), torch.randn(Fd, H, device=device, dtype=dtype)
    wd = torch.randn(H, Fd, device=device, dtype=dtype)
    x = torch.randn(B, S, H, device=device, dtype=dtype)
    with torch.no_grad():
        ms = _time_fn(lambda: F.linear(F.silu(F.linear(x, wg)) * F.linear(x, wu), wd), device)
    return {"bench": "dense_ffn_forward", "B": B, "S": S, "H": H, "F": Fd, "ms": ms}


def bench_token_conservation(device, dtype, seeds: int = 100, N=512, H=128, E=32, K=2):
    violations = 0
    for seed in range(seeds):
        torch.manual_seed(seed)
        x = torch.randn(N, H, device=device, dtype=dtype)
        w = (torch.randn(H, E, device=device) / H**0.5).to(dtype)
        idx, wt = moe_topk_route(x, w, K)
        counts = torch.bincount(idx.reshape(-1), minlength=E)
        ok = int(counts.sum()) == N * K and bool((idx >= 0).all()) and bool((idx < E).all())
        ok = ok and bool(torch.allclose(wt.float().sum(-1), torch.ones(N, device=device), atol=1e-2))
        ok = ok and all(len(set(r)) == K for r in idx[:16].tolist())
        violations += 0 if ok else 1
    return {"bench": "token_conservation", "seeds": seeds, "violations": violations}


def run_suite(device: str, dtype: torch.dtype):
    rows = []
    cfgs = ROUTER_CONFIGS + ([SPEC_ROUTER_CONFIG] if device == "cuda" else [])
    for cfg in cfgs:
        rows.append(bench_router_forward(*cfg, device, dtype))
        rows.append(bench_router_fwd_bwd(*cfg, device, dtype))
    for cfg in LAYER_CONFIGS:
        moe = bench_moe_layer(*cfg, device, dtype)
        dense = bench_dense_baseline(*cfg[:4], device, dtype)
        moe["dense_ms"] = dense["ms"]
        moe["moe_over_dense"] = moe["ms"] / max(dense["ms"], 1e-9)
        rows += [moe, dense]
    rows.append(bench_token_conservation(device, dtype))
    for r in rows:
        r["device"] = device
        r["dtype"] = str(dtype).replace("torch.", "")
    return rows


def _use_reference() -> None:
    """Rebind the benchmarked entry points to the unmodified reference package installed under baseline/_ref
    (its Triton router on a GPU, its Python expert loop), so both implementations run the same workloads here."""
    global moe_topk_route, DistributedMoELayer, _layer_topology
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "pkg").exists():
        raise SystemExit("baseline/_ref is not installed")
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref))
    for name in [m for m in sys.modules if m == "pkg" or m.startswith("pkg.")]:
        del sys.modules[name]
    from pkg.distributed.parallel_mesh import DistributedMoELayer as RefLayer
    from pkg.kernels.moe_router import moe_topk_route as ref_route

    from pkg.distributed.parallel_mesh import build_topology as ref_topology

    moe_topk_route, DistributedMoELayer = ref_route, RefLayer
    _layer_topology = lambda device: ref_topology(dp_size=1, ep_size=1, device_type=device)  # noqa: E731


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours",
                    help="'reference' runs the same suite on the unmodified reference under baseline/_ref")
    ap.add_argument("--cuda", action="store_true", help="also run the GPU suite")
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--csv", type=str, default=None)
    ap.add_argument("--dtype", choices=["bf16", "fp32"], default="bf16", help="input dtype of the GPU suite")
    ap.add_argument("--skip-cpu", action="store_true")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        _use_reference()
    rows = []
    if not args.skip_cpu:
        rows += run_suite("cpu", torch.float32)
    if args.cuda:
        if not torch.cuda.is_available():
            print("--cuda requested but no CUDA device is available", file=sys.stderr)
            return 2
        rows += run_suite("cuda", torch.bfloat16 if args.dtype == "bf16" else torch.float32)
    for r in rows:
        r["impl"] = args.impl
        print(json.dumps(r))
    if args.json:
        Path(args.json).write_text(json.dumps({"torch": torch.__version__, "results": rows}, indent=1))
    if args.csv:
        keys = sorted({k for r in rows for k in r})
        with open(args.csv, "w", newline="") as fh:
            wr = csv.DictWriter(fh, fieldnames=keys)
            wr.writeheader()
            wr.writerows(rows)
    bad = [r for r in rows if r["bench"] == "token_conservation" and r["violations"]]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
