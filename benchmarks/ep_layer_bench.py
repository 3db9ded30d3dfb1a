"""Expert-parallel MoE layer benchmark: one layer, forward and forward+backward, per transport.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/ep_layer_bench.py [--zipf 1.1]

Default shape is the expert-parallel layer of the benchmark spec: d=4096, 64 experts, F=1408, top-6, 8192 tokens
per rank, bf16, ep = N.  For every transport (``nccl``: all-gather / reduce-scatter; ``peer``: NVLink peer memory
with the dispatch pulled inside the first GEMM; ``peer-push``: the same with the combine pushed by the GEMM
epilogues) it reports the device time of the layer, and next to it the time of the same expert math on rows that are
already local (no transfers): the difference is the exposed dispatch + combine cost per layer, the number the
reference's design documents target at < 0.6-0.8 ms (docs/benchmarks.md:284-291) without measuring it.

Roofline per transport: ``max(expert FLOPs of this rank / measured bf16 peak, NVLink bytes into this GPU / link
rate)`` with the bytes counted from the row plan (rows whose token lives on another rank, once for the dispatch and
once for the combine; twice that for forward + backward) and ``--link-gbs`` as the per-direction link rate (default
770, the measured peer-copy rate of this pool; 900 nominal).  ``standalone`` times the two transfers as kernels of
their own (``gather_rows_peer`` / ``combine_rows_peer`` on the same plan) against bytes / link rate.

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
    ap.add_argument("--transports", default="nccl,peer-push,peer")
    ap.add_argument("--link-gbs", type=float, default=770.0)
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

    # ---- rooflines from the plan of the last forward --------------------------------------------------------
    peak = 1590.0
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.loads(pk.read_text()).get("bf16_tflops", peak))
    plan = layer._last_plan_holder.get("plan") if world > 1 else None
    if plan is not None:
        n_rows = int(plan.num_m_tiles) * 128
        rs = plan.row_slot[:n_rows]
        kept = rs >= 0
        remote = int((kept & ((rs // (T * K)) != rank)).sum())
        real = int(kept.sum())
        flops_fwd = 2.0 * real * 3 * H * F  # gate, up, down projections of the rows this rank serves
        link = args.link_gbs * 1e9
        x_bytes = remote * H * 2            # dispatch: token rows in;  combine: as many result rows out / in
        out["plan"] = {"rows_served": real, "rows_from_other_ranks": remote, "dispatch_bytes_in": x_bytes,
                       "combine_bytes": x_bytes, "expert_flops_fwd": flops_fwd, "bf16_peak_tflops": peak,
                       "link_gb_per_s": args.link_gbs}
        roof_f = max(flops_fwd / (peak * 1e12), 2 * x_bytes / link) * 1e3
        roof_fb = max(3 * flops_fwd / (peak * 1e12), 4 * x_bytes / link) * 1e3
        for red in ("roof_f", "roof_fb"):  # the slowest rank sets the layer time: take the largest roofline too
            t = torch.tensor([roof_f if red == "roof_f" else roof_fb], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if red == "roof_f":
                roof_f = float(t.item())
            else:
                roof_fb = float(t.item())
        out["roofline"] = {"fwd_ms": roof_f, "fwd_bwd_ms": roof_fb}
        for name, v in out["transports"].items():
            v["fwd_of_roofline"] = roof_f / v["fwd_ms"]
            v["fwd_bwd_of_roofline"] = roof_fb / v["fwd_bwd_ms"]
        # the two transfers as kernels of their own, on the same plan (pull transport: the result rows stay with
        # the expert's rank and the token's rank pulls them)
        if "peer" in out["transports"] and args.transports.split(",")[-1] == "peer":
            from composed_mixture_of_experts_engine_b200.ops import _ext
            from composed_mixture_of_experts_engine_b200.parallel import symm_peer

            ext = _ext.ext()
            pc = symm_peer._context(topo)
            lkey = (symm_peer._layer_key(layer), (layer._peer_forward_calls - 1) % max(1, topo.pp_size))
            xs = pc.shared("x", T * H * 2)
            srow = pc.per_layer(lkey, "slot_row", world * T * K * 4)
            yps = pc.per_layer(lkey, "yp", plan.cap_rows * H * 2)
            xp = torch.empty(plan.cap_rows, H, device=dev, dtype=torch.bfloat16)
            yv = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
            idx32 = layer.router.last_idx32.contiguous()
            w32 = layer.router.last_w32.detach().float().contiguous()
            erank = pc.expert_rank_table(E)
            d_ms = _median_ms(lambda: ext.gather_rows_peer(xs.ptrs(), T * K, K, plan.row_slot, None, xp,
                                                           plan.num_m_tiles, H), args.iters, args.warmup, dev)
            c_ms = _median_ms(lambda: ext.combine_rows_peer(yps.ptrs(), srow.ptrs(), idx32, erank, w32, yv, K,
                                                            rank * T * K, H, None), args.iters, args.warmup, dev)
            bt = torch.tensor([float(x_bytes)], device=dev, dtype=torch.float64)
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
            worst_bytes = float(bt.item())
            out["standalone"] = {
                "dispatch_ms": d_ms, "dispatch_of_nvlink_roofline": worst_bytes / link * 1e3 / d_ms,
                "combine_ms": c_ms, "combine_of_nvlink_roofline": worst_bytes / link * 1e3 / c_ms,
                "dispatch_gb_per_s_in": worst_bytes / 1e9 / d_ms * 1e3,
                "combine_gb_per_s_in": worst_bytes / 1e9 / c_ms * 1e3}

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
    if "standalone" in out:
        # how much of the transfers' stand-alone time the fused layer hides under the expert math
        from composed_mixture_of_experts_engine_b200.telemetry.logger import overlap_ratio

        comm = out["standalone"]["dispatch_ms"] + out["standalone"]["combine_ms"]
        for name, v in out["transports"].items():
            v["comm_compute_overlap_ratio_fwd"] = overlap_ratio(comm, lf, v["fwd_ms"])
    if world > 1 and "peer-push" in out["transports"]:
        # device timestamps of the fused GEMM1 (first / last row pulled, first / last MMA) of one more forward pass
        os.environ["CMOE_EP_TRANSPORT"], os.environ["CMOE_EP_PUSH"] = "auto", "1"
        layer.enable_timing(True)
        for _ in range(3):
            fwd()
        torch.cuda.synchronize()
        stamps = layer._last_plan_holder.get("pull_stamps")
        if stamps is not None:
            p0, p1, m0, m1 = (int(v) for v in stamps.tolist())
            out["fused_gemm1_timeline_us"] = {"pull_first_to_last": (p1 - p0) / 1e3, "mma_first_to_last": (m1 - m0) / 1e3,
                                              "first_mma_after_first_pull": (m0 - p0) / 1e3,
                                              "last_mma_after_last_pull": (m1 - p1) / 1e3,
                                              "overlap_ratio": layer.last_overlap_ratio}
        layer.enable_timing(False)
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
