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

    python benchmarks/loss_parity.py --device cuda --steps 200
    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/loss_parity.py --device cuda \
        [--transport nccl]

``--device cuda`` compares this package with itself: the attention decoder trained by the public ``Trainer`` in bf16
on the sm_100a kernels (fused optimizer with fp32 master weights; on several GPUs dp = ep = N with the peer-memory
or the NCCL transport) against the same decoder in fp32 on the PyTorch path on CPU (stock AdamW), from equal
weights on equal batches (the CPU run sees the union of all ranks' batches, which is what data parallelism
averages over).  Here the two sides compute the same function, so the curves must agree to bf16 rounding; the line
reports the largest loss gap and the largest relative gap of the gradient norms.
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


def _self_parity(a) -> None:
    """bf16 CUDA trainer (this package's kernels) against the fp32 CPU path of the same decoder."""
    import os

    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    if a.transport != "auto":
        os.environ["CMOE_EP_TRANSPORT"] = os.environ["CMOE_DP_TRANSPORT"] = a.transport
    import torch.distributed as dist

    from composed_mixture_of_experts_engine_b200.engine import Trainer, init_distributed
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    rank, world = init_distributed("cuda")

    def cfg(dtype, dp):
        return MoEConfig.from_dict({
            "model": dict(arch="moe_decoder", hidden_dim=256, num_layers=2, num_heads=4, num_experts=8, top_k=2,
                          ffn_dim=256, vocab_size=2048, sequence_length=256, dtype=dtype, aux_loss_coeff=0.01,
                          init_std=0.02),
            "training": dict(micro_batch_size=a.batch, gradient_accumulation_steps=1, global_batch_size=a.batch * dp,
                             max_steps=10 * a.steps, warmup_steps=0, learning_rate=a.lr, grad_clip=1.0, seed=3),
            "parallelism": dict(data_parallel=dp, expert_parallel=dp, ep_from_dp=True)})

    gpu = Trainer(cfg("bfloat16", world))
    V, S = 2048, 256
    pools = []
    for r in range(world):  # every rank's pool of batches, seen repeatedly so that the loss falls within the run
        gen = torch.Generator().manual_seed(100 + r)
        pools.append([(torch.randint(0, V, (a.batch, S), generator=gen), torch.randint(0, V, (a.batch, S), generator=gen))
                      for _ in range(4)])
    # the fp32 twin on CPU (rank 0 only): all experts in one process, the union of the ranks' batches per step
    cpu = None
    full_state = None
    if world > 1:
        # gather the expert shards so that rank 0 can assemble the whole model
        parts = [None] * world
        dist.all_gather_object(parts, {k: v.float().cpu() for k, v in gpu.model.state_dict().items()})
        full_state = {}
        for k in parts[0]:
            if k.rsplit(".", 1)[-1] in ("w13", "w2"):
                full_state[k] = torch.cat([p[k] for p in parts], dim=0)
            else:
                full_state[k] = parts[0][k]
    else:
        full_state = {k: v.float().cpu() for k, v in gpu.model.state_dict().items()}
    if rank == 0:
        from composed_mixture_of_experts_engine_b200.parallel import ParallelTopology

        c = cfg("float32", 1)
        d = c.to_dict()
        d["training"].update(micro_batch_size=a.batch * world, global_batch_size=a.batch * world)
        cpu = Trainer(MoEConfig.from_dict(d), device_type="cpu", topology=ParallelTopology(1, 0, 1, 1))
        cpu.model.load_state_dict(full_state)
        torch.set_num_threads(max(1, min(16, os.cpu_count() or 1)))
    l_gpu, l_cpu, n_gpu, n_cpu = [], [], [], []
    for i in range(a.steps):
        ids, tgt = pools[rank][i % 4]
        loss = gpu.train_step(ids, tgt).detach().clone()
        if world > 1:
            dist.all_reduce(loss)
            loss /= world
        l_gpu.append(float(loss))
        n_gpu.append(gpu.optimizer.grad_norm())
        if cpu is not None:
            ids_all = torch.cat([pools[r][i % 4][0] for r in range(world)])
            tgt_all = torch.cat([pools[r][i % 4][1] for r in range(world)])
            l_cpu.append(float(cpu.train_step(ids_all, tgt_all)))
            n_cpu.append(cpu.last_grad_norm)
        if world > 1:
            dist.barrier()  # the other ranks do not start the next device step while rank 0 is still on its CPU step
    if rank == 0:
        diffs = [abs(x - y) for x, y in zip(l_gpu, l_cpu)]
        rel_norm = [abs(x - y) / max(y, 1e-12) for x, y in zip(n_gpu, n_cpu)]
        print(json.dumps({
            "mode": "bf16 CUDA kernels vs fp32 CPU path of the same decoder", "n_gpus": world,
            "transport": ("peer memory" if a.transport == "auto" else a.transport) if world > 1 else "none",
            "steps": a.steps, "first_loss": [l_gpu[0], l_cpu[0]], "last_loss": [l_gpu[-1], l_cpu[-1]],
            "max_abs_loss_gap": max(diffs), "mean_abs_loss_gap": sum(diffs) / len(diffs),
            "max_rel_grad_norm_gap": max(rel_norm), "mean_rel_grad_norm_gap": sum(rel_norm) / len(rel_norm),
            "grad_norm_first_last": [[n_gpu[0], n_cpu[0]], [n_gpu[-1], n_cpu[-1]]]}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu",
                    help="cpu: against the unmodified reference in fp32; cuda: the bf16 kernels against this package's "
                         "own fp32 CPU path")
    ap.add_argument("--transport", choices=["auto", "nccl"], default="auto", help="--device cuda on several GPUs")
    a = ap.parse_args()
    if a.device == "cuda":
        _self_parity(a)
        return
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
