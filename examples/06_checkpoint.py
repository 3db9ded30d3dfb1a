"""Asynchronous two-tier checkpoints: save without blocking, retention, resume, remote fallback."""
import sys
import tempfile
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import torch
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.elastic import AsyncCheckpointer, LocalNVMeAdapter

torch.manual_seed(0)
model = nn.Sequential(nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 8))
opt = torch.optim.AdamW(model.parameters(), lr=1e-3)

with tempfile.TemporaryDirectory() as d:
    local, remote = LocalNVMeAdapter(f"{d}/nvme"), LocalNVMeAdapter(f"{d}/remote", use_odirect=False)
    ckpt = AsyncCheckpointer(local, remote, retention=2, workers=2)
    for step in range(1, 6):
        model(torch.randn(16, 64)).sum().backward()
        opt.step()
        opt.zero_grad()
        t0 = time.perf_counter()
        ckpt.save(model, opt, step)
        print(f"step {step}: save() returned after {1e3 * (time.perf_counter() - t0):.2f} ms "
              f"(last_commit_ms={ckpt.last_commit_ms:.2f})")
    ckpt.shutdown(drain=True)
    print("kept locally:", sorted({k.split('/')[1] for k in local.list('ckpts/')}), "| O_DIRECT used:",
          local.last_write_used_odirect)

    fresh = nn.Sequential(nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 8))
    fresh_opt = torch.optim.AdamW(fresh.parameters(), lr=1e-3)
    for k in local.list("ckpts/"):
        local.delete(k)  # lose the fast tier
    loader = AsyncCheckpointer(local, remote, workers=1)
    meta = loader.load(fresh, fresh_opt, loader.latest_step() or 5)
    loader.shutdown()
    same = all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), fresh.state_dict().values()))
    print("restored from the remote tier:", same, "| meta step", meta["step"], "schema", meta["schema_version"])
