#!/usr/bin/env python
"""Loss-curve parity with the unmodified reference on CPU (fp32): the reference's ``ToyMoEModel`` (installed under
``baseline/_ref``) and this package's ``ToyMoEModel`` start from the same weights, see the same synthetic token
batches and take the same ``torch.optim.AdamW`` steps; the script prints both curves' distance as one JSON line.

    python benchmarks/loss_parity.py --steps 200

The two layers do not compute the same function: the reference applies experts by row position after sorting on
the first routing slot only (pkg/distributed/moe_layer.py:318-336), this package applies
``y_t = sum_k w[t,k] * Expert_{idx[t,k]}(x_t)``.  Routers, norms, embedding and head agree exactly from equal
weights, so the first losses differ only by the expert mix (5.68 against 5.70 here) and the curves fall together
(200 steps: 2.28 against 2.42, largest gap 0.22); identical curves cannot be expected.
Reference recipe: cross entropy on fp32 logits, AdamW(betas=(0.9, 0.95)), global-norm clip 1.0
(train.py:207-212,297-323 of the reference).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

DIMS = dict(vocab_size=256, hidden_dim=64, num_layers=2, num_experts=8, top_k=2, ffn_dim=128, sequence_length=32,
            capacity_factor=1.25, dtype="float32")


def _cfg_dict(batch: int) -> dict:
    return {
        "model": dict(DIMS),
        "training": dict(global_batch_size=batch, micro_batch_size=batch, learning_rate=3e-4, weight_decay=0.1,
                         grad_clip=1.0, max_steps=10000, warmup_steps=0, gradient_accumulation_steps=1),
        "parallelism": dict(data_parallel=1, expert_parallel=1, tensor_parallel=1, pipeline_parallel=1),
        "checkpoint": dict(local_dir="/tmp/parity-ckpt", remote_uri="file:///tmp/parity-remote"),
    }


def _build_ours(batch: int):
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    from composed_mixture_of_experts_engine_b200.models import build_model
    from composed_mixture_of_experts_engine_b200.parallel import build_topology
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict(_cfg_dict(batch))
    topo = build_topology(dp_size=1, ep_size=1, tp_size=1, pp_size=1, device_type="cpu")
    return build_model(cfg, topo)


def _build_reference(batch: int):
    # the reference package is called `pkg`, like this repository's compatibility package: make the installed
    # reference the one that `import pkg` finds
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(REF))
    for name in [m for m in sys.modules if m == "pkg" or m.startswith("pkg.")]:
        del sys.modules[name]
    from pkg.distributed import build_topology
    from pkg.models.moe import build_model
    from pkg.utils.config import MoEConfig

    assert str(Path(sys.modules["pkg"].__file__).resolve()).startswith(str(REF.resolve()))
    cfg = MoEConfig.from_dict(_cfg_dict(batch))
    topo = build_topology(dp_size=1, ep_size=1, tp_size=1, pp_size=1, device_type="cpu")
    return build_model(cfg, topo)


def _copy_weights(ref, ours) -> None:
    with torch.no_grad():
        ours.embed.weight.copy_(ref.embed.weight)
        ours.norm.weight.copy_(ref.norm.weight)
        ours.lm_head.weight.copy_(ref.lm_head.weight)
        for rb, ob in zip(ref.blocks, ours.blocks):
            ob.norm.weight.copy_(rb.norm.weight)
            ob.moe.router.gate_w.copy_(rb.moe.router.gate_w)
            for re_, oe in zip(rb.moe.experts, ob.moe.experts):
                # this package's experts are live views into the layer's stacked weights
                oe.w_gate.weight.copy_(re_.w_gate.weight)
                oe.w_up.weight.copy_(re_.w_up.weight)
                oe.w_down.weight.copy_(re_.w_down.weight)


def _train(model, batches, lr: float):
    V = DIMS["vocab_size"]
    optim = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=0.1, betas=(0.9, 0.95))
    losses = []
    for ids, tgt in batches:
        optim.zero_grad(set_to_none=True)
        logits = model(ids)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, V).float(), tgt.reshape(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optim.step()
        losses.append(float(loss.detach()))
    return losses


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--lr", type=float, default=3e-4)
    a = ap.parse_args()
    if not (REF / "pkg").is_dir():
        print(json.dumps({"unavailable": "baseline/_ref is not installed"}))
        return
    torch.manual_seed(0)
    torch.set_num_threads(1)
    ours = _build_ours(a.batch)
    ref = _build_reference(a.batch)
    _copy_weights(ref, ours)
    gen = torch.Generator().manual_seed(0)
    V, S = DIMS["vocab_size"], DIMS["sequence_length"]
    # a small pool of batches seen repeatedly, so that the loss actually falls within the run
    pool = [(torch.randint(0, V, (a.batch, S), generator=gen), torch.randint(0, V, (a.batch, S), generator=gen))
            for _ in range(4)]
    batches = [pool[i % len(pool)] for i in range(a.steps)]
    l_ref = _train(ref, batches, a.lr)
    l_ours = _train(ours, batches, a.lr)
    diffs = [abs(x - y) for x, y in zip(l_ref, l_ours)]
    print(json.dumps({
        "steps": a.steps, "first_loss": [l_ref[0], l_ours[0]], "last_loss": [l_ref[-1], l_ours[-1]],
        "max_abs_diff": max(diffs), "max_abs_diff_first_20": max(diffs[:20]),
        "mean_abs_diff": sum(diffs) / len(diffs),
    }))


if __name__ == "__main__":
    main()
