"""Expert-parallel MoE layer benchmark: one layer, forward and forward+backward, per transport.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/ep_layer_bench.py [--zipf 1.1]

Default shape is the expert-parallel layer of the benchmark spec: d=4096, 64 experts, F=1408, top-6, 8192 tokens
per rank, bf16, ep = N.  For every transport (``nccl``: all-gather / reduce-scatter; ``peer``: NVLink peer memory
with the dispatch pulled inside the first GEMM; ``peer-push``: the same with the combine pushed by the GEMM
epilogues) it reports the device time of the layer, and next to it the time of the same expert math on rows that are
already local (no transfers): the difference is the exposed dispatch + combine cost per layer, the number the
reference's design documents target at < 0.6-0.8 ms (docs/benchmarks.md:284-291) without measuring it.

All times are CUDA-event times on the launching stream, median of ``--iters`` after ``--warmup`` runs, maximum over
ranks; an L2-sized buffer is overwritten between iterations.  ``--zipf s`` skews the routing (expert popularity
~ 1 / rank^s) by shifting the inputs along the gate columns.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _median_ms(fn, iters: int, warmup: int, device) -> float:
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        if dist.is_initialized():
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    t = torch.tensor([times[len(times) // 2]], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=6)
    ap.add_argument("--tokens", type=int, default=8192, help="tokens per rank")
    ap.add_argument("--zipf", type=float, default=0.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--transports", default="nccl,peer,peer-push")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world)

    if args.zipf > 0:  # skewed routing: size the row buffers for the worst case so that nothing is dropped
        os.environ["CMOE_EP_BUFFER_FACTOR"] = str(world)
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status, overflow_counter
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology

    H, F, E, K, T = args.hidden, args.ffn, args.experts, args.top_k, args.tokens
    topo = build_topology(1, world, device_type="cuda")
    dev = topo.device
    torch.manual_seed(1234)
    layer = DistributedMoELayer(H, F, E, K, topology=topo, dtype=torch.bfloat16).to(dev)
    torch.manual_seed(100 + rank)
    x = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    if args.zipf > 0:
        # skew the routing through the inputs: a shift along every expert's gate column proportional to the log of
        # its target popularity moves the logits by about that much (the columns are nearly orthogonal)
        with torch.no_grad():
            pop = 1.0 / torch.arange(1, E + 1, device=dev, dtype=torch.float32) ** args.zipf
            bias = torch.log(pop / pop.sum())
            g = layer.router.gate_w.float()  # [H, E]
            shift = (g / (g * g).sum(0, keepdim=True) * bias[None, :]).sum(1)
            x = (x.float() + shift[None, :]).to(torch.bfloat16)
    x.requires_grad_()
    dy = torch.randn(T, H, device=dev, dtype=torch.bfloat16)

    def fwd():
        with torch.no_grad():
            return layer(x)

    def fwd_bwd():
        y = layer(x)
        y.backward(dy)
        x.grad = None

    out = {"bench": "ep_layer", "n_gpus": world, "hidden": H, "ffn": F, "experts": E, "top_k": K,
           "tokens_per_rank": T, "zipf": args.zipf, "dtype": "bf16", "timing": "CUDA events, median, max over ranks",
           "transports": {}}
    for name in args.transports.split(","):
        if world == 1 and name != "nccl":
            continue
        os.environ["CMOE_EP_TRANSPORT"] = "nccl" if name == "nccl" else "auto"
        os.environ["CMOE_EP_PUSH"] = "1" if name == "peer-push" else "0"
        f = _median_ms(fwd, args.iters, args.warmup, dev)
        fb = _median_ms(fwd_bwd, args.iters, args.warmup, dev)
        check_status(dev)
        out["transports"][name] = {"fwd_ms": f, "fwd_bwd_ms": fb}

    # the same amount of expert math on rows that are already here: a layer without expert parallelism that holds
    # this rank's share of the experts and sees as many (token, expert) rows as this rank processed above
    holder = layer._last_plan_holder
    rows = int(holder["plan"].num_m_tiles) * 128 if holder and "plan" in holder else T * K
    n_local = layer.w13.shape[0]
    k_loc = min(K, n_local)
    t_loc = max(128, rows // k_loc)
    local_layer = DistributedMoELayer(H, F, n_local, k_loc, dtype=torch.bfloat16).to(dev)
    xl = (torch.randn(t_loc, H, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
    dyl = torch.randn(t_loc, H, device=dev, dtype=torch.bfloat16)

    def loc_fwd():
        with torch.no_grad():
            return local_layer(xl)

    def loc_fwd_bwd():
        local_layer(xl).backward(dyl)
        xl.grad = None

    lf = _median_ms(loc_fwd, args.iters, args.warmup, dev)
    lfb = _median_ms(loc_fwd_bwd, args.iters, args.warmup, dev)
    out["local_rows"] = t_loc * k_loc
    out["local_math"] = {"fwd_ms": lf, "fwd_bwd_ms": lfb}
    for name, v in out["transports"].items():
        v["exposed_dispatch_combine_fwd_us"] = (v["fwd_ms"] - lf) * 1e3
        v["exposed_dispatch_combine_fwd_bwd_us"] = (v["fwd_bwd_ms"] - lfb) * 1e3
    out["rows_dropped_for_buffer_space"] = int(overflow_counter(dev).item()) if world > 1 else 0
    out["rows_this_rank"] = rows
    if rank == 0:
        print(json.dumps(out))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
