"""NVLink peer-memory bandwidth as this package's own kernels see it: plain P2P loads and stores, no library copy.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/p2p_bandwidth.py [--mbytes 256]

Every rank holds one buffer of ``--mbytes`` MiB in symmetric memory.  Measured per rank, all ranks at the same time
(so every link is loaded in both directions, as in the expert-parallel exchange):

* ``pull 1<-1``: 16-byte loads of one neighbour's whole buffer into local memory (``peer_allgather`` with a single source);
* ``pull 1<-all``: the same from all ``N - 1`` peers (one launch);
* ``push 1->all``: 16-byte stores of the local buffer into every peer's buffer (``push_shard``);
* ``row pull``: the expert-parallel dispatch pattern, whole rows of 4 KiB gathered from random rows of random
  peers by one warp per row (``gather_rows_peer``).

Times are CUDA events on the launching stream, median of ``--iters`` launches after warm-up, maximum over ranks;
bandwidth counts the bytes that cross NVLink into (pull) or out of (push) one GPU.  These are the link-rate
denominators of the fused compute + collective rooflines.  The reference has no counterpart (it only calls NCCL).
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
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
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
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world < 2:
        print(json.dumps({"bench": "p2p_bandwidth", "unavailable": "needs at least two GPUs"}))
        return 0
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", rank=rank, world_size=world)

    from composed_mixture_of_experts_engine_b200.ops import _ext
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.parallel import build_topology, symm

    ext = _ext.ext()
    topo = build_topology(1, world, device_type="cuda")
    dev = topo.device
    sg = symm.group_for(topo, "ep")
    nbytes = args.mbytes << 20
    buf = sg.alloc("p2p.bench", nbytes)
    src = buf.view(torch.bfloat16, nbytes // 2)
    src.normal_()
    ptrs = buf.ptrs()
    torch.cuda.synchronize()
    dist.barrier()

    out = {"bench": "p2p_bandwidth", "n_gpus": world, "mbytes_per_buffer": args.mbytes,
           "timing": "CUDA events, median, max over ranks; all ranks transfer at the same time"}
    gb = nbytes / 1e9

    one = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    nxt = [ptrs[(rank + 1) % world]]
    ms = _median_ms(lambda: ext.peer_allgather(nxt, nbytes, one), args.iters, args.warmup, dev)
    out["pull_1_from_1"] = {"ms": ms, "gb_per_s": gb / ms * 1e3}

    others = [ptrs[(rank + 1 + i) % world] for i in range(world - 1)]
    allb = torch.empty(nbytes * (world - 1), dtype=torch.uint8, device=dev)
    ms = _median_ms(lambda: ext.peer_allgather(others, nbytes, allb), args.iters, args.warmup, dev)
    out["pull_1_from_all"] = {"ms": ms, "gb_per_s": gb * (world - 1) / ms * 1e3}

    # push: every rank writes its own 1/world slice of the buffer into the same slice of every peer (disjoint slices)
    shard = (nbytes // 2 // world) // 8 * 8
    ms = _median_ms(lambda: ext.push_shard(ptrs, rank, rank * shard, shard, src), args.iters, args.warmup, dev)
    out["push_1_to_all"] = {"ms": ms, "gb_per_s": shard * 2 * (world - 1) / 1e9 / ms * 1e3,
                            "bytes_per_peer": shard * 2}

    # row pull: rows of H bf16 elements from random rows of random peers (never the local buffer)
    H = 2048
    rows_per_buf = nbytes // (2 * H)
    n_rows = rows_per_buf  # pull as many rows as one buffer holds
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    peer = (rank + 1 + torch.randint(0, world - 1, (n_rows,), generator=g)) % world
    row = torch.randint(0, rows_per_buf, (n_rows,), generator=g)
    slot = (peer * rows_per_buf + row).to(torch.int32).to(dev)
    dst = torch.empty(n_rows, H, dtype=torch.bfloat16, device=dev)
    tiles = torch.tensor([n_rows // 128], dtype=torch.int32, device=dev)
    ms = _median_ms(lambda: ext.gather_rows_peer(ptrs, rows_per_buf, 1, slot, None, dst, tiles, H), args.iters,
                    args.warmup, dev)
    out["row_pull_4KiB_rows"] = {"ms": ms, "gb_per_s": (n_rows // 128 * 128) * H * 2 / 1e9 / ms * 1e3}

    check_status(dev)
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
