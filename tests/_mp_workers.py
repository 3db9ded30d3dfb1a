"""Worker functions for the multi-process (gloo, CPU) tests.  Each takes (rank, world, port, queue, *args)."""

from __future__ import annotations

import os
import sys
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _init(rank: int, world: int, port: int, backend: str = "gloo"):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), GLOO_SOCKET_IFNAME="lo")
    if backend == "nccl":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


def run(fn_name: str, rank: int, world: int, port: int, queue, args, backend: str = "gloo"):
    import torch
    import torch.distributed as dist

    torch.set_num_threads(1)
    try:
        _init(rank, world, port, backend)
        out = globals()[fn_name](rank, world, *args)
        queue.put((rank, "ok", out))
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------
def ep_layer(rank, world, capacity_dropping):
    """Expert-parallel layer on `world` ranks: output and gradients vs the single-rank layer holding all experts."""
    import torch

    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology

    H, F, E, K, N = 16, 32, 8, 2, 24
    topo = build_topology(1, world, device_type="cpu")
    torch.manual_seed(0)
    full = DistributedMoELayer(H, F, E, K, capacity_factor=0.25, capacity_dropping=capacity_dropping)
    layer = DistributedMoELayer(H, F, E, K, topology=topo, capacity_factor=0.25, capacity_dropping=capacity_dropping)
    mine = topo.experts_on_this_rank(E)
    with torch.no_grad():
        layer.router.gate_w.copy_(full.router.gate_w)
        layer.w13.copy_(full.w13[mine[0]:mine[-1] + 1])
        layer.w2.copy_(full.w2[mine[0]:mine[-1] + 1])
    torch.manual_seed(100 + rank)  # every rank routes its own tokens
    x = torch.randn(N, H, requires_grad=True)
    y = layer(x)
    y.pow(2).sum().backward()
    x2 = x.detach().clone().requires_grad_(True)
    y2 = full(x2)
    y2.pow(2).sum().backward()
    # expert-weight gradients: the sharded layer sees the tokens of ALL ranks; sum the oracle over ranks
    import torch.distributed as dist

    g13 = full.w13.grad.clone()
    dist.all_reduce(g13)
    return {
        "y": float((y - y2).abs().max()),
        "dx": float((x.grad - x2.grad).abs().max()),
        "dw13": float((layer.w13.grad - g13[mine[0]:mine[-1] + 1]).abs().max()),
        "dgate": float((layer.router.gate_w.grad - full.router.gate_w.grad).abs().max()),
        "dropped": layer.last_dropped_token_fraction,
    }


def tp_linears(rank, world):
    """Column -> SiLU -> Row over tp=world vs the unsharded computation, forward and backward."""
    import torch
    import torch.nn.functional as F

    from composed_mixture_of_experts_engine_b200.parallel import (ColumnParallelLinear, RowParallelLinear,
                                                                  build_topology)

    topo = build_topology(1, 1, tp_size=world, device_type="cpu")
    torch.manual_seed(0)
    Wc, Wr = torch.randn(32, 16), torch.randn(16, 32)
    col = ColumnParallelLinear(16, 32, bias=False, topology=topo, gather_output=False)
    row = RowParallelLinear(32, 16, bias=False, topology=topo)
    sh = 32 // world
    with torch.no_grad():
        col.weight.copy_(Wc[rank * sh:(rank + 1) * sh])
        row.weight.copy_(Wr[:, rank * sh:(rank + 1) * sh])
    x = torch.randn(3, 5, 16, requires_grad=True)
    y = row(F.silu(col(x)))
    y.sum().backward()
    x2 = x.detach().clone().requires_grad_(True)
    y2 = F.linear(F.silu(F.linear(x2, Wc)), Wr)
    y2.sum().backward()
    gathered = ColumnParallelLinear(16, 32, bias=True, topology=topo, gather_output=True)
    with torch.no_grad():
        gathered.weight.copy_(Wc[rank * sh:(rank + 1) * sh])
    full_out = gathered(x.detach())
    return {"y": float((y - y2).abs().max()), "dx": float((x.grad - x2.grad).abs().max()),
            "gather": float((full_out - F.linear(x.detach(), Wc)).abs().max()),
            "row_full_input": float((row(F.silu(F.linear(x.detach(), Wc))) - y2.detach()).abs().max())}


def sp_linears(rank, world):
    """Sequence-parallel column/row pair: all-gather -> GEMM and GEMM -> reduce-scatter vs unsharded."""
    import torch
    import torch.nn.functional as F

    from composed_mixture_of_experts_engine_b200.parallel import (ColumnParallelLinear, RowParallelLinear,
                                                                  build_topology, gather_from_sequence_parallel,
                                                                  scatter_to_sequence_parallel)

    topo = build_topology(1, 1, tp_size=world, device_type="cpu")
    torch.manual_seed(0)
    Wc, Wr = torch.randn(32, 16), torch.randn(16, 32)
    x_full = torch.randn(2, 8, 16)
    col = ColumnParallelLinear(16, 32, bias=False, topology=topo, gather_output=False, sequence_parallel=True)
    row = RowParallelLinear(32, 16, bias=False, topology=topo, sequence_parallel=True)
    sh = 32 // world
    with torch.no_grad():
        col.weight.copy_(Wc[rank * sh:(rank + 1) * sh])
        row.weight.copy_(Wr[:, rank * sh:(rank + 1) * sh])
    x = x_full.clone().requires_grad_(True)
    xs = scatter_to_sequence_parallel(x, topo)
    ys = row(F.silu(col(xs)))
    y = gather_from_sequence_parallel(ys, topo)
    y.sum().backward()
    x2 = x_full.clone().requires_grad_(True)
    y2 = F.linear(F.silu(F.linear(x2, Wc)), Wr)
    y2.sum().backward()
    fused = scatter_to_sequence_parallel(x_full, topo, next_weight=Wc)
    return {"shape": list(xs.shape), "y": float((y - y2).abs().max()), "dx": float((x.grad - x2.grad).abs().max()),
            "fused": float((fused - F.linear(x_full, Wc)).abs().max())}


def pp_1f1b(rank, world, m):
    """`world` pipeline stages, each y = W_s x: outputs and the input/weight gradients vs the chained computation."""
    import torch
    import torch.nn as nn

    from composed_mixture_of_experts_engine_b200.parallel import PipelineStage, build_topology

    topo = build_topology(1, 1, pp_size=world, device_type="cpu")
    torch.manual_seed(0)
    Ws = [torch.randn(6, 6) / 2 for _ in range(world)]
    mod = nn.Linear(6, 6, bias=False)
    with torch.no_grad():
        mod.weight.copy_(Ws[rank])
    stage = PipelineStage(rank, world, mod, topo)
    mbs = [torch.randn(3, 6) for _ in range(m)]  # same seed on every rank
    outs, losses = stage.run_1f1b_distributed(mbs if rank == 0 else [], loss_fn=lambda o: o.pow(2).sum(),
                                              num_microbatches=m, activation_shape=(3, 6),
                                              activation_dtype=torch.float32, device=torch.device("cpu"))
    ref_w = [w.clone().requires_grad_(True) for w in Ws]
    total = 0
    ref_outs = []
    for x in mbs:
        h = x
        for w in ref_w:
            h = h @ w.t()
        ref_outs.append(h)
        total = total + h.pow(2).sum()
    total.backward()
    res = {"dw": float((mod.weight.grad - ref_w[rank].grad).abs().max()), "n_out": len(outs), "n_loss": len(losses)}
    if rank == world - 1:
        res["out"] = max(float((a - b).abs().max()) for a, b in zip(outs, ref_outs))
    return res


def trainer_steps(rank, world, config_path, steps):
    """The public Trainer on `world` gloo ranks (dp = ep = world, ep carved from dp)."""
    import torch

    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_yaml(config_path)
    tr = Trainer(cfg, device_type="cpu")
    gen = torch.Generator().manual_seed(rank)
    ids, tgt = tr.synthetic_batch(gen, pinned=False)
    losses = [float(tr.train_step(ids, tgt)) for _ in range(steps)]
    gate = tr.model.blocks[0].moe.router.gate_w.detach().clone()
    import torch.distributed as dist

    ref = gate.clone()
    dist.broadcast(ref, src=0)
    return {"losses": losses, "gate_sync": float((gate - ref).abs().max()), "ep": tr.topology.ep_size,
            "local_experts": tr.model.blocks[0].moe.local_expert_ids}


def train_main_tp(rank, world, tmp_dir):
    """``train.py`` itself on `world` gloo ranks with tensor parallelism and sequence parallelism OFF: the
    tensor-parallel peers of one data replica must be fed the same tokens (the row-parallel all-reduce sums partial
    products of ONE activation), which shows as identical logged losses on all of them."""
    import json

    import yaml

    import train as train_main_module

    cfg = {
        "model": dict(arch="moe_decoder", hidden_dim=32, num_layers=2, num_heads=2, num_experts=4, top_k=2,
                      ffn_dim=64, vocab_size=128, sequence_length=16, dtype="float32", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=1, global_batch_size=2, max_steps=4,
                         warmup_steps=0, learning_rate=1e-3, log_interval=1, ckpt_interval=0, seed=0),
        "parallelism": dict(data_parallel=1, expert_parallel=1, tensor_parallel=world, pipeline_parallel=1,
                            ep_from_dp=True, sequence_parallel=False),
        "checkpoint": dict(local_dir=f"{tmp_dir}/ck{rank}", remote_uri=f"file://{tmp_dir}/remote{rank}"),
        "telemetry": dict(log_dir=f"{tmp_dir}/logs", tensorboard_dir=f"{tmp_dir}/tb",
                          json_path=f"{tmp_dir}/logs/step.jsonl"),
    }
    path = f"{tmp_dir}/tp{rank}.yaml"
    with open(path, "w") as f:
        yaml.safe_dump(cfg, f)
    # train.main() initialises (and at the end destroys) the process group itself
    import torch.distributed as dist

    if dist.is_initialized():
        # a fresh rendezvous port agreed on over the old group: re-using the old port races with rank 0 closing
        # the store that the other ranks may still be connected to
        box = [None]
        if rank == 0:
            from tests.conftest import find_free_port

            box[0] = find_free_port()
        dist.broadcast_object_list(box, src=0)
        dist.barrier()
        dist.destroy_process_group()
        os.environ["MASTER_PORT"] = str(box[0])
    rc = train_main_module.main(["--config", path, "--cpu", "--no-wandb"])
    rows = [json.loads(l) for l in open(f"{tmp_dir}/logs/step.rank{rank}.jsonl") if l.strip().startswith("{")]
    return {"rc": rc, "losses": [r["loss"] for r in rows if "loss" in r]}


def moe_layer_tp(rank, world):
    """MoE layer with the experts sliced on the FFN width over tp=world ranks vs the unsliced layer: output, token
    gradient, router gate gradient (needs the all-reduce of the partial gate-weight gradients) and weight slices."""
    import torch

    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology

    H, F, E, K, N = 16, 32, 4, 2, 20
    topo = build_topology(1, 1, tp_size=world, device_type="cpu")
    torch.manual_seed(0)
    full = DistributedMoELayer(H, F, E, K)
    layer = DistributedMoELayer(H, F, E, K, topology=topo)
    fl = F // world
    lo, hi = rank * fl, (rank + 1) * fl
    with torch.no_grad():
        layer.router.gate_w.copy_(full.router.gate_w)
        layer.w13.copy_(torch.cat([full.w13[:, lo:hi], full.w13[:, F + lo:F + hi]], dim=1))
        layer.w2.copy_(full.w2[:, :, lo:hi])
    torch.manual_seed(7)  # the same tokens on every tensor-parallel rank
    x = torch.randn(N, H, requires_grad=True)
    y = layer(x)
    y.pow(2).sum().backward()
    x2 = x.detach().clone().requires_grad_(True)
    y2 = full(x2)
    y2.pow(2).sum().backward()
    g13 = torch.cat([full.w13.grad[:, lo:hi], full.w13.grad[:, F + lo:F + hi]], dim=1)
    return {"y": float((y - y2).abs().max()), "dx": float((x.grad - x2.grad).abs().max()),
            "dgate": float((layer.router.gate_w.grad - full.router.gate_w.grad).abs().max()),
            "dw13": float((layer.w13.grad - g13).abs().max()),
            "dw2": float((layer.w2.grad - full.w2.grad[:, :, lo:hi]).abs().max())}


def trainer_hybrid(rank, world, dp, ep, tp, pp, steps):
    """The public Trainer with tensor (+ sequence) and pipeline parallelism on gloo ranks: tiny fp32 decoder, 1F1B over
    4 microbatches.  Returns the per-step losses this rank saw (only the last pipeline stage sees them)."""
    import torch

    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict({
        "model": dict(arch="moe_decoder", hidden_dim=64, num_layers=4, num_heads=4, num_experts=4, top_k=2,
                      ffn_dim=128, vocab_size=256, sequence_length=32, dtype="float32", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=4, global_batch_size=8 * dp, max_steps=50,
                         warmup_steps=0, learning_rate=2e-3, grad_clip=1.0, seed=0),
        "parallelism": dict(data_parallel=dp, expert_parallel=ep, tensor_parallel=tp, pipeline_parallel=pp,
                            ep_from_dp=True, sequence_parallel=tp > 1)})
    tr = Trainer(cfg, device_type="cpu")
    gen = torch.Generator().manual_seed(tr.topology.dp_rank)  # replicas of one model shard see the same data
    ids, tgt = tr.synthetic_batch(gen, pinned=False)
    losses = [float(tr.train_step(ids, tgt)) for _ in range(steps)]
    blk = tr.model.blocks[0]
    replicated = {"norm": blk.norm.weight, "attn_norm": blk.attn_norm.weight, "gate": blk.moe.router.gate_w}
    return {"losses": losses, "pp_rank": tr.topology.pp_rank, "tp_rank": tr.topology.tp_rank,
            "dp_rank": tr.topology.dp_rank, "last": tr.topology.is_last_pp_stage(),
            "n_blocks": len(tr.model.blocks),
            "replicated": {k: v.detach().double().flatten()[:64].tolist() for k, v in replicated.items()}}


def trainer_ep_axis(rank, world, dp, ep, steps):
    """Expert parallelism as a mesh axis of its own (``ep_from_dp=False``): every expert-parallel rank draws its own
    data, so the dense parameters are replicated over dp x ep ranks and must stay identical on all of them."""
    import torch

    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict({
        "model": dict(arch="moe_decoder", hidden_dim=32, num_layers=2, num_heads=2, num_experts=4, top_k=2,
                      ffn_dim=64, vocab_size=128, sequence_length=16, dtype="float32", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=1, global_batch_size=2 * dp * ep,
                         max_steps=50, warmup_steps=0, learning_rate=5e-3, grad_clip=1.0, seed=0),
        "parallelism": dict(data_parallel=dp, expert_parallel=ep, tensor_parallel=1, pipeline_parallel=1,
                            ep_from_dp=False)})
    tr = Trainer(cfg, device_type="cpu")
    gen = torch.Generator().manual_seed(tr.topology.data_rank)  # every data replica its own tokens
    losses = []
    for _ in range(steps):
        ids, tgt = tr.synthetic_batch(gen, pinned=False)
        losses.append(float(tr.train_step(ids, tgt)))
    blk = tr.model.blocks[0]
    dense = {"gate": blk.moe.router.gate_w, "norm": blk.norm.weight, "wqkv": blk.attn.wqkv.weight,
             "embed": tr.model.embed.weight}
    return {"losses": losses, "data_rank": tr.topology.data_rank, "data_replicas": tr.topology.data_replicas,
            "dense": {k: v.detach().double().flatten()[:96].tolist() for k, v in dense.items()},
            "expert": blk.moe.w13.detach().double().flatten()[:32].tolist()}


def _elastic_cfg(dp, ep):
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    return MoEConfig.from_dict({
        "model": dict(arch="moe_decoder", hidden_dim=32, num_layers=2, num_heads=2, num_experts=8, top_k=2,
                      ffn_dim=48, vocab_size=128, sequence_length=16, dtype="float32", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=1, global_batch_size=2 * dp, max_steps=50,
                         warmup_steps=0, learning_rate=5e-3, grad_clip=1.0, seed=0),
        "parallelism": dict(data_parallel=dp, expert_parallel=ep, tensor_parallel=1, pipeline_parallel=1,
                            ep_from_dp=True)})


def _expert_fingerprints(tr, num_experts):
    """sha256 of every locally held expert's weights and Adam moments, keyed by global expert id, plus the
    fingerprints of a few dense tensors and their moments."""
    import hashlib

    import torch

    def sha(t):
        return hashlib.sha256(t.detach().contiguous().cpu().numpy().tobytes()).hexdigest()

    mine = tr.topology.experts_on_this_rank(num_experts)
    state = tr.optimizer.state
    out = {"experts": {}, "dense": {}}
    for li, layer in enumerate(tr.model.moe_layers()):
        for pname, p in (("w13", layer.w13), ("w2", layer.w2)):
            st = state[p]
            for j, e in enumerate(mine):
                out["experts"][f"{li}.{pname}.{e}"] = [sha(p[j]), sha(st["exp_avg"][j]), sha(st["exp_avg_sq"][j])]
    blk = tr.model.blocks[0]
    for name, p in (("gate", blk.moe.router.gate_w), ("wqkv", blk.attn.wqkv.weight), ("embed", tr.model.embed.weight)):
        st = state[p]
        out["dense"][name] = [sha(p), sha(st["exp_avg"]), sha(st["exp_avg_sq"])]
    return out


def elastic_save(rank, world, ckpt_dir, steps):
    """Phase 1 of the shrink test: dp = ep = world (ep carved from dp), a few steps, one checkpoint."""
    import torch

    from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import ElasticConfig, ElasticTrainerHarness
    from composed_mixture_of_experts_engine_b200.engine import Trainer

    tr = Trainer(_elastic_cfg(world, world), device_type="cpu")
    gen = torch.Generator().manual_seed(tr.topology.data_rank)
    for _ in range(steps):
        ids, tgt = tr.synthetic_batch(gen, pinned=False)
        tr.train_step(ids, tgt)
    h = ElasticTrainerHarness(ElasticConfig(ckpt_dir, None, async_workers=1), tr.topology)
    h.checkpoint(tr.model, tr.optimizer, steps)
    h.shutdown()
    return _expert_fingerprints(tr, 8)


def elastic_resume(rank, world, ckpt_dir):
    """Phase 2: half as many ranks build the same model on the smaller mesh and resume from the files of phase 1."""
    import math

    import torch

    from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import ElasticConfig, ElasticTrainerHarness
    from composed_mixture_of_experts_engine_b200.engine import Trainer

    tr = Trainer(_elastic_cfg(world, world), device_type="cpu")
    h = ElasticTrainerHarness(ElasticConfig(ckpt_dir, None, async_workers=1), tr.topology)
    step = h.resume(tr.model, tr.optimizer, 8)
    fp = _expert_fingerprints(tr, 8)
    ids, tgt = tr.synthetic_batch(torch.Generator().manual_seed(tr.topology.data_rank), pinned=False)
    loss = float(tr.train_step(ids, tgt))  # the re-assembled optimizer state is usable
    h.shutdown()
    return {"step": step, "fp": fp, "finite": math.isfinite(loss), "mine": tr.topology.experts_on_this_rank(8)}


def _fused_optimizer_on_cpu(model, topo):
    """The fused optimizer's flat groups built on CPU tensors (its step needs the CUDA kernels, its state layout,
    sharding and state dict do not), with recognisable values in master / m / v: element i of a dense parameter
    holds tag(name) + i / n; element i of expert e's slice holds tag(name) + 10 e + i / n."""
    import zlib

    import torch

    from composed_mixture_of_experts_engine_b200.ops.optim import FusedAdamW, _FlatGroup
    from composed_mixture_of_experts_engine_b200.parallel.mesh import ddp_process_group, edp_process_group

    params = list(model.named_parameters())
    dense = [(n, p) for n, p in params if not getattr(p, "is_expert_param", False)]
    expert = [(n, p) for n, p in params if getattr(p, "is_expert_param", False)]
    groups = [
        _FlatGroup("dense", [p for _, p in dense], torch.float32, [True] * len(dense),
                   shard_group=ddp_process_group(topo), topology=None, param_names=[n for n, _ in dense]),
        _FlatGroup("expert", [p for _, p in expert], torch.float32, [True] * len(expert),
                   shard_group=edp_process_group(topo), topology=None, param_names=[n for n, _ in expert])]
    opt = FusedAdamW(groups, lr=1e-3)
    mine = topo.experts_on_this_rank(8)

    def expected(name, p):
        tag = float(zlib.crc32(name.encode()) % 997)
        if getattr(p, "is_expert_param", False):
            per = p[0].numel()
            return torch.cat([tag + 10.0 * e + torch.arange(per, dtype=torch.float32) / per for e in mine])
        return tag + torch.arange(p.numel(), dtype=torch.float32) / p.numel()

    return opt, expected


def fused_reshard_save(rank, world, ckpt_dir):
    """dp = ep = world (carved): dense state sharded over all ranks, expert state unsharded per owner."""
    import torch

    from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import ElasticConfig, ElasticTrainerHarness
    from composed_mixture_of_experts_engine_b200.engine import Trainer

    tr = Trainer(_elastic_cfg(world, world), device_type="cpu", build_optim=False)
    opt, expected = _fused_optimizer_on_cpu(tr.model, tr.topology)
    for g in opt.groups:
        full = torch.zeros(g.numel)
        for n, off, p in zip(g.param_names, g.offsets, g.params):
            full[off:off + p.numel()] = expected(n, p)
        sl = slice(g.shard_lo, g.shard_lo + g.shard_numel)
        g.master.copy_(full[sl])
        g.m.copy_(full[sl] + 0.25)
        g.v.copy_(full[sl] + 0.5)
    opt.step_count = 11
    h = ElasticTrainerHarness(ElasticConfig(ckpt_dir, None, async_workers=1), tr.topology)
    h.checkpoint(tr.model, opt, 11)
    h.shutdown()
    return {"dense_shard_world": opt.groups[0].shard_world, "expert_shard_world": opt.groups[1].shard_world}


def fused_reshard_load(rank, world, ckpt_dir):
    import torch

    from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import ElasticConfig, ElasticTrainerHarness
    from composed_mixture_of_experts_engine_b200.engine import Trainer

    tr = Trainer(_elastic_cfg(world, world), device_type="cpu", build_optim=False)
    opt, expected = _fused_optimizer_on_cpu(tr.model, tr.topology)
    h = ElasticTrainerHarness(ElasticConfig(ckpt_dir, None, async_workers=1), tr.topology)
    step = h.resume(tr.model, opt, 8)
    h.shutdown()
    worst = 0.0
    for g in opt.groups:
        full = torch.zeros(g.numel)
        for n, off, p in zip(g.param_names, g.offsets, g.params):
            full[off:off + p.numel()] = expected(n, p)
        sl = slice(g.shard_lo, g.shard_lo + g.shard_numel)
        covered = torch.zeros(g.numel, dtype=torch.bool)
        for off, p in zip(g.offsets, g.params):
            covered[off:off + p.numel()] = True  # alignment padding between parameters carries no state
        mask = covered[sl]
        for t, shift in ((g.master, 0.0), (g.m, 0.25), (g.v, 0.5)):
            worst = max(worst, float(((t - (full[sl] + shift)) * mask).abs().max()))
    return {"step": step, "opt_step": opt.step_count, "worst": worst, "dense_shard_world": opt.groups[0].shard_world}


# -------------------------------------------------------------------------------------------------- GPU workers
def _set_transport(transport):
    """"nccl", "auto" (peer memory, results pushed by the GEMM epilogues), "auto-pull" (peer memory, pulled) or
    "auto-debug" (as "auto" with the debug-mode checks switched on)."""
    push = "0" if transport.endswith("-pull") else "1"
    os.environ["CMOE_EP_PUSH"] = os.environ["CMOE_TP_PUSH"] = push
    if transport.endswith("-debug"):  # row-plan index checks + guard bands around the symmetric buffers
        os.environ["CMOE_DEBUG_BOUNDS"] = "1"
    os.environ["CMOE_EP_TRANSPORT"] = transport.replace("-pull", "").replace("-debug", "")


def gpu_ep_layer(rank, world, transport):
    """bf16 expert-parallel layer on `world` GPUs vs the same layer with all experts on one GPU."""
    import torch
    import torch.distributed as dist

    _set_transport(transport)
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology

    H, F, E, K, N = 256, 512, 16, 4, 1024
    topo = build_topology(1, world, device_type="cuda")
    dev = topo.device
    torch.manual_seed(0)
    full = DistributedMoELayer(H, F, E, K, dtype=torch.bfloat16).to(dev)
    layer = DistributedMoELayer(H, F, E, K, topology=topo, dtype=torch.bfloat16).to(dev)
    mine = topo.experts_on_this_rank(E)
    with torch.no_grad():
        layer.router.gate_w.copy_(full.router.gate_w)
        layer.w13.copy_(full.w13[mine[0]:mine[-1] + 1])
        layer.w2.copy_(full.w2[mine[0]:mine[-1] + 1])
    out = {}
    for it in range(2):  # twice: buffers and flags are reused
        torch.manual_seed(100 + rank + 10 * it)
        x = torch.randn(N, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        dy = torch.randn(N, H, device=dev, dtype=torch.bfloat16)
        for l in (layer, full):
            l.zero_grad(set_to_none=True)
        y = layer(x)
        y.backward(dy)
        x2 = x.detach().clone().requires_grad_(True)
        y2 = full(x2)
        y2.backward(dy)
        g13 = full.w13.grad.float().clone()
        dist.all_reduce(g13)
        rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
        out[f"y{it}"] = rel(y, y2)
        out[f"dx{it}"] = rel(x.grad, x2.grad)
        out[f"dw13_{it}"] = rel(layer.w13.grad, g13[mine[0]:mine[-1] + 1])
        out[f"dgate{it}"] = rel(layer.router.gate_w.grad, full.router.gate_w.grad)
        if it == 1:
            # the same inputs once more: bit-identical results (no sum in the exchange or in the expert GEMMs depends
            # on the order in which peers or CTAs arrive), so any difference is a race
            keep = [t.detach().clone() for t in (y, x.grad, layer.w13.grad, layer.w2.grad, layer.router.gate_w.grad)]
            layer.zero_grad(set_to_none=True)
            x3 = x.detach().clone().requires_grad_(True)
            y3 = layer(x3)
            y3.backward(dy)
            again = (y3, x3.grad, layer.w13.grad, layer.w2.grad, layer.router.gate_w.grad)
            out["replay"] = max(float((a.float() - b.float()).abs().max()) for a, b in zip(keep, again))
    check_status(dev)
    if transport.endswith("-debug"):  # nothing (this rank or a peer) wrote outside a symmetric buffer
        from composed_mixture_of_experts_engine_b200.parallel import symm

        symm.group_for(topo, "ep").verify_guards()
    return out


def gpu_moe_sequence_shard(rank, world, ep, tp):
    """The MoE layer under tensor + sequence parallelism fed sequence shards (peer memory over the ep x tp block,
    FFN slices routed as experts of their own) vs the unsliced layer with all experts on one GPU."""
    import torch
    import torch.distributed as dist

    os.environ["CMOE_EP_TRANSPORT"] = "auto"
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer, build_topology
    from composed_mixture_of_experts_engine_b200.parallel.mesh import tp_process_group

    H, F, E, K, T = 256, 512, 8, 2, 1024  # T tokens per data replica (= per expert-parallel rank)
    topo = build_topology(ep, ep, tp_size=tp, device_type="cuda", ep_from_dp=True)
    dev = topo.device
    torch.manual_seed(0)
    full = DistributedMoELayer(H, F, E, K, dtype=torch.bfloat16).to(dev)
    layer = DistributedMoELayer(H, F, E, K, topology=topo, dtype=torch.bfloat16).to(dev)
    mine = topo.experts_on_this_rank(E)
    e0, e1 = mine[0], mine[-1] + 1
    fl, j = F // tp, topo.tp_rank
    with torch.no_grad():
        layer.router.gate_w.copy_(full.router.gate_w)
        layer.w13[:, :fl].copy_(full.w13[e0:e1, j * fl:(j + 1) * fl])          # gate rows of this slice
        layer.w13[:, fl:].copy_(full.w13[e0:e1, F + j * fl:F + (j + 1) * fl])  # up rows of this slice
        layer.w2.copy_(full.w2[e0:e1, :, j * fl:(j + 1) * fl])
    rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
    out = {"fused": bool(layer.fused_sequence_shard_path(torch.empty(1, H, device=dev, dtype=torch.bfloat16)))}
    T_l = T // tp
    for it in range(2):  # twice: buffers, flags and in-flight slots are reused
        xs, dys = [], []
        for d in range(ep):  # every data replica's tokens, so that each rank can form the reference gradients
            torch.manual_seed(100 + d + 10 * it)
            xs.append(torch.randn(T, H, device=dev, dtype=torch.bfloat16))
            dys.append(torch.randn(T, H, device=dev, dtype=torch.bfloat16))
        d = topo.dp_rank
        x = xs[d][j * T_l:(j + 1) * T_l].clone().requires_grad_(True)
        dy = dys[d][j * T_l:(j + 1) * T_l]
        for l in (layer, full):
            l.zero_grad(set_to_none=True)
        y = layer(x, sequence_shard=True)
        y.backward(dy)
        gate_grad = layer.router.gate_w.grad.float().clone()
        dist.all_reduce(gate_grad, group=tp_process_group(topo))  # partial per sequence shard
        x_all = torch.cat(xs).requires_grad_(True)
        y_all = full(x_all)
        y_all.backward(torch.cat(dys))
        lo = d * T + j * T_l
        out[f"y{it}"] = rel(y, y_all[lo:lo + T_l])
        out[f"dx{it}"] = rel(x.grad, x_all.grad[lo:lo + T_l])
        g13, g2 = full.w13.grad, full.w2.grad
        want13 = torch.cat([g13[e0:e1, j * fl:(j + 1) * fl], g13[e0:e1, F + j * fl:F + (j + 1) * fl]], dim=1)
        out[f"dw13_{it}"] = rel(layer.w13.grad, want13)
        out[f"dw2_{it}"] = rel(layer.w2.grad, g2[e0:e1, :, j * fl:(j + 1) * fl])
        # the reference's gate gradient covers all replicas' tokens; sum this replica's over the data replicas too
        if ep > 1:
            from composed_mixture_of_experts_engine_b200.parallel.mesh import ep_process_group

            dist.all_reduce(gate_grad, group=ep_process_group(topo))
        out[f"dgate{it}"] = rel(gate_grad, full.router.gate_w.grad)
    check_status(dev)
    return out


def gpu_trainer(rank, world, transport, steps):
    """Trainer on `world` GPUs (dp = ep = world, sharded optimizer): finite decreasing loss, replicas in sync."""
    import torch
    import torch.distributed as dist

    os.environ["CMOE_EP_TRANSPORT"] = transport
    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict({
        "model": dict(arch="moe_decoder", hidden_dim=256, num_layers=2, num_heads=4, num_experts=8, top_k=2,
                      ffn_dim=256, vocab_size=2048, sequence_length=256, dtype="bfloat16", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=2, max_steps=100, warmup_steps=0,
                         learning_rate=1e-3),
        "parallelism": dict(data_parallel=world, expert_parallel=world, ep_from_dp=True)})
    tr = Trainer(cfg)
    ids, tgt = tr.synthetic_batch(torch.Generator().manual_seed(rank))
    losses = [float(tr.train_step(ids, tgt)) for _ in range(steps)]
    check_status(tr.device)
    w = tr.model.blocks[0].attn.wqkv.weight.detach().float().clone()
    ref = w.clone()
    dist.broadcast(ref, src=0)
    return {"losses": losses, "sync": float((w - ref).abs().max()), "ep": tr.topology.ep_size,
            "n_local": len(tr.model.blocks[0].moe.local_expert_ids)}


def gpu_trainer_hybrid(rank, world, dp, ep, tp, pp, steps):
    """bf16 Trainer on GPUs with pipeline (and optionally tensor / expert) parallelism: NCCL 1F1B, fused optimizer."""
    import torch

    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict({
        "model": dict(arch="moe_decoder", hidden_dim=256, num_layers=4, num_heads=4, num_experts=8, top_k=2,
                      ffn_dim=256, vocab_size=2048, sequence_length=256, dtype="bfloat16", aux_loss_coeff=0.01,
                      init_std=0.02),
        "training": dict(micro_batch_size=2, gradient_accumulation_steps=4, global_batch_size=8 * dp, max_steps=100,
                         warmup_steps=0, learning_rate=1e-3, grad_clip=1.0),
        "parallelism": dict(data_parallel=dp, expert_parallel=ep, tensor_parallel=tp, pipeline_parallel=pp,
                            ep_from_dp=True, sequence_parallel=tp > 1)})
    tr = Trainer(cfg)
    ids, tgt = tr.synthetic_batch(torch.Generator().manual_seed(tr.topology.dp_rank))
    losses = [float(tr.train_step(ids, tgt)) for _ in range(steps)]
    check_status(tr.device)
    # parameters that every tensor-parallel rank holds whole must stay bit-identical on all of them: their gradients
    # are partial sums per sequence shard, summed over the group before the update
    blk = tr.model.blocks[0]
    whole = {"norm": blk.norm.weight, "attn_norm": blk.attn_norm.weight, "gate": blk.moe.router.gate_w}
    if tr.model.embed is not None:
        whole["embed"] = tr.model.embed.weight
    if tr.model.lm_head is not None:
        whole["lm_head"] = tr.model.lm_head.weight
    return {"losses": losses, "last": tr.topology.is_last_pp_stage(), "n_blocks": len(tr.model.blocks),
            "tp_rank": tr.topology.tp_rank, "pp_rank": tr.topology.pp_rank,
            "whole": {k: v.detach().double().flatten()[:256].tolist() for k, v in whole.items()},
            "fused_sp_moe": bool(getattr(blk.moe.router.gate_w, "sequence_parallel_grad", False))}


def gpu_tp_sp(rank, world, transport="auto"):
    """Sequence-parallel column -> SiLU -> row pair over tp=world GPUs on the peer-memory path vs unsharded."""
    import torch
    import torch.nn.functional as F

    _set_transport(transport)
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status
    from composed_mixture_of_experts_engine_b200.parallel import (ColumnParallelLinear, RowParallelLinear,
                                                                  build_topology, gather_from_sequence_parallel,
                                                                  scatter_to_sequence_parallel)

    topo = build_topology(1, 1, tp_size=world, device_type="cuda")
    dev = topo.device
    torch.manual_seed(0)
    B, S, Din, Dmid = 2, 512, 256, 512
    Wc = (torch.randn(Dmid, Din, device=dev) / Din**0.5).to(torch.bfloat16)
    Wr = (torch.randn(Din, Dmid, device=dev) / Dmid**0.5).to(torch.bfloat16)
    x_full = torch.randn(B, S, Din, device=dev, dtype=torch.bfloat16)
    col = ColumnParallelLinear(Din, Dmid, bias=False, topology=topo, gather_output=False, sequence_parallel=True,
                               dtype=torch.bfloat16, device=dev)
    row = RowParallelLinear(Dmid, Din, bias=False, topology=topo, sequence_parallel=True, dtype=torch.bfloat16,
                            device=dev)
    sh = Dmid // world
    with torch.no_grad():
        col.weight.copy_(Wc[rank * sh:(rank + 1) * sh])
        row.weight.copy_(Wr[:, rank * sh:(rank + 1) * sh])
    out = {}
    for it in range(2):
        x = x_full.clone().requires_grad_(True)
        col.zero_grad(set_to_none=True)
        row.zero_grad(set_to_none=True)
        ys = row(F.silu(col(scatter_to_sequence_parallel(x, topo))))
        y = gather_from_sequence_parallel(ys, topo)
        y.float().pow(2).sum().backward()
        x2 = x_full.clone().float().requires_grad_(True)
        wc, wr = Wc.float().requires_grad_(True), Wr.float().requires_grad_(True)
        y2 = F.linear(F.silu(F.linear(x2, wc)), wr)
        y2.pow(2).sum().backward()
        rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
        out[f"y{it}"] = rel(y, y2)
        out[f"dx{it}"] = rel(x.grad, x2.grad)
        out[f"dwc{it}"] = rel(col.weight.grad, wc.grad[rank * sh:(rank + 1) * sh])
        out[f"dwr{it}"] = rel(row.weight.grad, wr.grad[:, rank * sh:(rank + 1) * sh])
    check_status(dev)
    return out


def pp_announced(rank, world, m):
    """The reference's calling convention (tests/test_pipeline_parallel.py:174-243): only stage 0 holds the
    micro-batches, later stages pass an empty list and no shape; count, shape and dtype travel in a header."""
    import torch
    import torch.nn as nn

    from composed_mixture_of_experts_engine_b200.parallel import PipelineStage, build_topology

    topo = build_topology(dp_size=1, ep_size=1, tp_size=1, pp_size=world, device_type="cpu")
    mod = nn.Linear(6, 4 if rank == 0 else 4, bias=False) if rank == 0 else nn.Linear(4, 4, bias=False)
    with torch.no_grad():
        mod.weight.fill_(0.5)
    stage = PipelineStage(rank, world, mod, topo)
    mbs = [torch.ones(3, 6) for _ in range(m)] if rank == 0 else []
    outs, losses = stage.run_1f1b_distributed(mbs, loss_fn=lambda o: o.sum())
    expect = 6 * 0.5 * (4 * 0.5) ** (world - 1)
    return {"n_out": len(outs), "n_loss": len(losses),
            "out": max((float((o - expect).abs().max()) for o in outs), default=0.0),
            "shape": list(outs[0].shape) if outs else [],
            "grad": float(mod.weight.grad.abs().sum()) if mod.weight.grad is not None else 0.0}

