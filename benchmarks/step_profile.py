"""Kernel breakdown of one training step (torch profiler, device time per kernel), on one or several GPUs.

    python benchmarks/step_profile.py [--micro-batch 4] [--accum 1]
    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/step_profile.py \
        [--config configs/mixtral_8x7b.yaml --mesh 1,1,2,2 --layers 16 --micro-batch 1 --accum 8] [--rank 3]

Builds the public ``Trainer`` (default: the headline OLMoE-shaped configuration with dp = ep = N, ep carved from
dp), runs three warm-up steps, times one step with CUDA events without the profiler, then wraps one more step in
``torch.profiler`` on one rank (``--rank``, default 0; the others run the same step unprofiled) and prints the
kernels by self device time.  The figures explain the ``bench.py`` numbers; a time taken under the profiler is never
a benchmark value.  Output of this script is what ``profiles/train_step_breakdown.md`` is written from.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=str(ROOT / "configs" / "olmoe_1b7b.yaml"))
    ap.add_argument("--mesh", default=None, metavar="DP,EP,TP,PP", help="default: dp = ep = world, tp = pp = 1")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--rank", type=int, default=0, help="the rank that runs under the profiler")
    ap.add_argument("--top", type=int, default=45)
    args = ap.parse_args()

    import torch.distributed as dist

    from composed_mixture_of_experts_engine_b200.engine import Trainer, init_distributed
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    rank, world = init_distributed("cuda")
    d = MoEConfig.from_yaml(args.config).to_dict()
    if args.mesh:
        dp, ep, tp, pp = (int(v) for v in args.mesh.split(","))
    else:
        dp, ep, tp, pp = world, world, 1, 1
    d["parallelism"].update(data_parallel=dp, expert_parallel=ep, tensor_parallel=tp, pipeline_parallel=pp,
                            ep_from_dp=True, sequence_parallel=tp > 1, pipeline_microbatches=args.accum if pp > 1 else 0)
    if args.layers > 0:
        d["model"]["num_layers"] = args.layers
    d["training"].update(micro_batch_size=args.micro_batch, gradient_accumulation_steps=args.accum,
                         global_batch_size=args.micro_batch * args.accum * dp, warmup_steps=0, max_steps=1000)
    tr = Trainer(MoEConfig.from_dict(d))
    ids, tgt = tr.synthetic_batch(torch.Generator().manual_seed(tr.topology.dp_rank))
    ids, tgt = ids.cuda(), tgt.cuda()
    for _ in range(3):
        tr.train_step(ids, tgt)
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    tr.train_step(ids, tgt)
    e1.record()
    torch.cuda.synchronize()
    who = args.rank if world > 1 else 0
    if rank == who:
        print(f"step {e0.elapsed_time(e1):.1f} ms without the profiler; rank {rank} of {world}, mesh dp{dp} ep{ep} "
              f"tp{tp} pp{pp}, {args.micro_batch} x {args.accum} sequences of {tr.seq} tokens per rank")
    if dist.is_initialized():
        dist.barrier()
    if rank == who:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            tr.train_step(ids, tgt)
            torch.cuda.synchronize()
        rows = [(ev.self_device_time_total, ev.count, ev.key) for ev in prof.key_averages()
                if ev.self_device_time_total > 0]
        rows.sort(reverse=True)
        total = sum(r[0] for r in rows)
        print(f"sum of kernel self times {total / 1000:.1f} ms")
        for t, c, k in rows[:args.top]:
            print(f"{t / 1000:9.2f} ms {100 * t / total:5.1f}% x{c:5d}  {k[:110]}")
    else:
        tr.train_step(ids, tgt)
        torch.cuda.synchronize()
    check_status(tr.device)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
