"""Worker of the chaos tests: a tiny data-parallel training loop on CPU/gloo that checkpoints every step.

Launched by torchrun with restarts.  Environment knobs (all host-side faults; no GPU is involved):
  CHAOS_DIR          working directory (checkpoints, per-rank JSONL logs)
  CHAOS_STEPS        total steps
  CHAOS_KILL_RANK    rank that SIGKILLs itself ...
  CHAOS_KILL_STEP    ... at this step, in restart generation 0 only  (-1: never)
  CHAOS_STALL_S      the local store's first put() sleeps this long (storage stall)
"""

from __future__ import annotations

import hashlib
import json
import os
import signal
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch
import torch.distributed as dist
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.elastic import AsyncCheckpointer, LocalNVMeAdapter
from composed_mixture_of_experts_engine_b200.engine import elastic_generation_store


def sha(model: nn.Module) -> str:
    h = hashlib.sha256()
    for k, v in sorted(model.state_dict().items()):
        h.update(k.encode())
        h.update(v.detach().cpu().numpy().tobytes())
    return h.hexdigest()


def main() -> int:
    work = Path(os.environ["CHAOS_DIR"])
    steps = int(os.environ.get("CHAOS_STEPS", "8"))
    kill_rank = int(os.environ.get("CHAOS_KILL_RANK", "-1"))
    kill_step = int(os.environ.get("CHAOS_KILL_STEP", "-1"))
    stall = float(os.environ.get("CHAOS_STALL_S", "0"))
    generation = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0"))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    # rendezvous keys private to this restart generation (a restarted worker must not read its predecessor's)
    dist.init_process_group("gloo", store=elastic_generation_store(rank, world), rank=rank, world_size=world)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
    opt = torch.optim.SGD(model.parameters(), lr=0.05)

    class Store(LocalNVMeAdapter):
        stalled = False

        def put(self, key, payload):
            if stall > 0 and not Store.stalled:
                Store.stalled = True
                time.sleep(stall)
            super().put(key, payload)

        def put_torch(self, key, obj):
            if stall > 0 and not Store.stalled:
                Store.stalled = True
                time.sleep(stall)
            super().put_torch(key, obj)

    ckpt = AsyncCheckpointer(Store(str(work / "ckpts")), None, retention=100, workers=1)
    log = (work / f"rank{rank}_gen{generation}.jsonl").open("a", buffering=1)
    start, cum_tokens = 0, 0
    # all ranks agree on the resume step: the newest step that EVERY rank has on disk
    mine = ckpt.latest_step()
    t = torch.tensor([mine if mine is not None else -1])
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    latest = int(t.item())
    if latest >= 0:
        meta = ckpt.load(model, opt, latest, rank=rank)
        start = latest + 1
        cum_tokens = int(meta.get("cum_tokens", 0))
        log.write(json.dumps({"event": "resume", "step": latest, "sha": sha(model), "want_sha": meta.get("sha"),
                              "generation": generation}) + "\n")
    tokens_per_step = 8
    for step in range(start, steps):
        if generation == 0 and rank == kill_rank and step == kill_step:
            os.kill(os.getpid(), signal.SIGKILL)  # a host-side process death
        g = torch.Generator().manual_seed(1000 * step + rank)
        x, y = torch.randn(tokens_per_step, 16, generator=g), torch.randn(tokens_per_step, 4, generator=g)
        loss = (model(x) - y).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        for p in model.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        cum_tokens += tokens_per_step
        t0 = time.perf_counter()
        ckpt.save(model, opt, step, rank=rank, extra_meta={"sha": sha(model), "cum_tokens": cum_tokens})
        blocked_ms = (time.perf_counter() - t0) * 1e3
        ckpt._q.join()  # the next step's resume point must be on disk before a possible kill
        log.write(json.dumps({"event": "step", "step": step, "loss": float(loss), "cum_tokens": cum_tokens,
                              "generation": generation, "save_blocked_ms": blocked_ms}) + "\n")
    ckpt.shutdown(drain=True)
    log.write(json.dumps({"event": "done", "sha": sha(model), "generation": generation}) + "\n")
    log.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
