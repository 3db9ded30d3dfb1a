"""Sequence-parallel tensor-parallel linears: all-gather -> GEMM and GEMM -> reduce-scatter, fused against library.

    torchrun --nnodes=1 --nproc-per-node TP --master-addr 127.0.0.1 benchmarks/tp_layer_bench.py

Default shapes are the attention projections of the Mixtral-shaped configuration at tp = 2: one sequence of 4096
tokens, d = 4096, column layer 4096 -> 6144 (q, k, v; 3072 per rank), row layer 4096 -> 4096 (2048 input features
per rank), bf16.  Arms:

* ``fused``: ``parallel/symm_tp.py``: the gather runs inside the tcgen05 GEMM (row-pull warps, P2P loads), the
  reduce-scatter is the GEMM epilogue's P2P row push plus a local fp32 sum;
* ``library``: NCCL ``all_gather_into_tensor`` + ``torch.matmul`` (cuBLAS) and ``torch.matmul`` +
  ``reduce_scatter_tensor`` - what the reference's call sites amount to once repaired
  (pkg/distributed/tensor_parallel.py:128,201-206; sequence_parallel.py:131,165).

Per op: CUDA-event time (median, max over ranks, L2 flushed between launches), the roofline
``max(FLOPs / measured bf16 peak, NVLink bytes per GPU / link rate)`` and achieved / roofline.  ``--link-gbs`` is
the per-direction link rate used (default 770, the measured peer-copy rate of this pool; 900 nominal).
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
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    t = torch.tensor([times[len(times) // 2]], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--col-out", type=int, default=6144, help="output features of the column layer (all ranks)")
    ap.add_argument("--row-in", type=int, default=4096, help="input features of the row layer (all ranks)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world < 2:
        print(json.dumps({"bench": "tp_layer", "unavailable": "needs at least two GPUs"}))
        return 0
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", rank=rank, world_size=world)

    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.parallel import build_topology, symm_tp
    from composed_mixture_of_experts_engine_b200.parallel.mesh import tp_process_group

    topo = build_topology(1, 1, tp_size=world, device_type="cuda")
    dev, group = topo.device, tp_process_group(topo)
    B, S, H, tp = args.batch, args.seq, args.hidden, world
    S_l, out_l, in_l = S // tp, args.col_out // tp, args.row_in // tp
    bf = torch.bfloat16
    torch.manual_seed(rank)
    x_shard = torch.randn(B, S_l, H, device=dev, dtype=bf)
    w_col = (torch.randn(out_l, H, device=dev) * 0.02).to(bf)
    x_full_sliced = torch.randn(B, S, in_l, device=dev, dtype=bf)
    w_row = (torch.randn(H, in_l, device=dev) * 0.02).to(bf)
    peak = 1590.0
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.loads(pk.read_text()).get("bf16_tflops", peak))

    gathered = torch.empty(tp * B * S_l, H, device=dev, dtype=bf)
    rs_out = torch.empty(B * S_l, H, device=dev, dtype=bf)

    def lib_ag_gemm():
        dist.all_gather_into_tensor(gathered, x_shard.view(B * S_l, H), group=group)
        return torch.matmul(gathered, w_col.t())

    def lib_gemm_rs():
        part = torch.matmul(x_full_sliced.view(B * S, in_l), w_row.t())
        dist.reduce_scatter_tensor(rs_out, part, group=group)
        return rs_out

    def fused_ag_gemm():
        with torch.no_grad():
            return symm_tp.allgather_linear(x_shard, w_col, topo)

    def fused_gemm_rs():
        with torch.no_grad():
            return symm_tp.linear_reduce_scatter(x_full_sliced, w_row, topo)

    link = args.link_gbs * 1e9
    rows = B * S
    ops = {
        "allgather_gemm": dict(flops=2.0 * rows * H * out_l, nvlink_bytes=(tp - 1) * B * S_l * H * 2,
                               fused=fused_ag_gemm, library=lib_ag_gemm),
        "gemm_reduce_scatter": dict(flops=2.0 * rows * in_l * H, nvlink_bytes=(tp - 1) * B * S_l * H * 2,
                                    fused=fused_gemm_rs, library=lib_gemm_rs),
    }
    out = {"bench": "tp_layer", "n_gpus": world, "batch": B, "seq": S, "hidden": H, "col_out": args.col_out,
           "row_in": args.row_in, "dtype": "bf16", "link_gb_per_s": args.link_gbs, "bf16_peak_tflops": peak,
           "timing": "CUDA events, median, max over ranks, L2 flushed between launches", "ops": {}}
    for name, op in ops.items():
        roof_ms = max(op["flops"] / (peak * 1e12), op["nvlink_bytes"] / link) * 1e3
        row = {"flops": op["flops"], "nvlink_bytes_in_per_gpu": op["nvlink_bytes"], "roofline_ms": roof_ms}
        for arm in ("fused", "library"):
            ms = _median_ms(op[arm], args.iters, args.warmup, dev)
            row[arm] = {"ms": ms, "of_roofline": roof_ms / ms}
        row["fused_vs_library"] = row["library"]["ms"] / row["fused"]["ms"]
        out["ops"][name] = row
    check_status(dev)
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
