"""``Trainer``: the public training API (what ``train.py`` and ``bench.py`` drive).

One object owns the topology, the model, the optimizer and the step function:

    trainer = Trainer(cfg)                     # cfg: MoEConfig
    loss = trainer.train_step(ids, targets)    # ids/targets: [micro_batch * accum, S] int64, CPU (pinned) or device
    trainer.close()

``train_step`` copies the batch to the device (asynchronously when it is pinned), runs
``gradient_accumulation_steps`` microbatches (or the 1F1B pipeline schedule when pipeline_parallel > 1), adds
the load-balance and z losses, clips by global norm, applies AdamW and returns the mean loss as a device
tensor, without waiting for the GPU on the host.  Counterpart of the hot loop in the reference's
train.py:284-323, minus its per-step host synchronisations (``.item()`` per microbatch, ``:320``).
"""

from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .models import build_model
from .models.decoder import MoEDecoder, finalize_sequence_parallel_grads
from .models.moe import DTYPE_MAP
from .ops.optim import FusedAdamW, build_optimizer
from .parallel.data_parallel import apply_fsdp2
from .parallel.mesh import ParallelTopology, build_topology
from .parallel.pipeline_parallel import PipelineStage
from .utils.config import MoEConfig

__all__ = ["Trainer", "init_distributed", "elastic_generation_store", "lr_at"]


def init_distributed(device_type: Optional[str] = None) -> Tuple[int, int]:
    """Join the process group described by the torchrun environment; returns (rank, world).  No-op for world 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        use_cuda = torch.cuda.is_available() and device_type != "cpu"
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1))))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        store = elastic_generation_store(rank, world)
        if store is not None:
            kwargs["store"] = store
        dist.init_process_group(backend="nccl" if use_cuda else "gloo", rank=rank, world_size=world, **kwargs)
    return rank, world


def elastic_generation_store(rank: int, world: int):
    """Under a TorchElastic launcher that restarts workers (``TORCHELASTIC_RESTART_COUNT`` set), a rendezvous store
    whose keys are private to this restart generation; ``None`` otherwise.

    The launcher's store outlives a worker generation.  A restarted worker that rendezvouses under the same keys
    can read the address its dead predecessor's peer published and then fails to connect ("connectFullMesh ...
    Connection refused"); prefixing the keys with the generation makes every restart start from an empty namespace."""
    gen = os.environ.get("TORCHELASTIC_RESTART_COUNT")
    addr, port = os.environ.get("MASTER_ADDR"), os.environ.get("MASTER_PORT")
    if gen is None or not addr or not port:
        return None
    from datetime import timedelta

    agent_hosts_store = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False").lower() in ("1", "true")
    base = dist.TCPStore(addr, int(port), world, is_master=(rank == 0 and not agent_hosts_store),
                         timeout=timedelta(seconds=300), multi_tenant=True)
    return dist.PrefixStore(f"generation{gen}", base)


def lr_at(step: int, base_lr: float, warmup_steps: int, max_steps: int) -> float:
    """Linear warm-up then cosine decay to 10 % of the base rate (reference train.py:108-113)."""
    if warmup_steps > 0 and step < warmup_steps:
        return base_lr * (step + 1) / warmup_steps
    span = max(1, max_steps - warmup_steps)
    progress = min(1.0, max(0.0, (step - warmup_steps) / span))
    return base_lr * (0.1 + 0.9 * 0.5 * (1.0 + math.cos(math.pi * progress)))


def fit_parallelism(cfg: MoEConfig, world: int) -> Tuple[int, int, int, int, bool]:
    """(dp, ep, tp, pp, ep_from_dp) that fits ``world`` ranks, shrinking dp (then ep) like the reference's
    train.py:173-186 when the configured product does not match."""
    par = cfg.parallelism
    tp, pp = par.tensor_parallel, par.pipeline_parallel
    if world == 1:
        return 1, 1, 1, 1, par.ep_from_dp
    if par.world_size == world:
        return par.data_parallel, par.expert_parallel, tp, pp, par.ep_from_dp
    if world % (tp * pp) != 0:
        tp, pp = 1, 1
    rest = world // (tp * pp)
    if par.ep_from_dp:
        dp = rest
        ep = math.gcd(par.expert_parallel, dp)
        while ep > 1 and cfg.model.num_experts % ep != 0:
            ep -= 1
        return dp, max(ep, 1), tp, pp, True
    ep = math.gcd(par.expert_parallel, rest)
    return rest // ep, ep, tp, pp, False


class _AttachAux(torch.autograd.Function):
    """Identity on ``x`` that also back-propagates a unit gradient into the scalar ``aux`` (a loss term that
    lives on a pipeline stage whose output is an activation, not a loss)."""

    @staticmethod
    def forward(ctx, x, aux):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g, g.new_ones(())


class Trainer:
    def __init__(self, cfg: MoEConfig, device_type: Optional[str] = None, topology: Optional[ParallelTopology] = None,
                 build_optim: bool = True):
        self.cfg = cfg
        use_cuda = torch.cuda.is_available() and device_type != "cpu"
        self.rank, self.world = init_distributed("cuda" if use_cuda else "cpu")
        if topology is None:
            dp, ep, tp, pp, carved = fit_parallelism(cfg, self.world)
            topology = build_topology(dp, ep, tp, pp, device_type="cuda" if use_cuda else "cpu", ep_from_dp=carved)
        self.topology = topology
        self.device = topology.device
        torch.manual_seed(cfg.training.seed + 1000 * topology.pp_rank + 17 * topology.tp_rank
                          + (topology.ep_rank if topology.ep_size > 1 else 0) * 100003)
        self.dtype = DTYPE_MAP.get(cfg.model.dtype, torch.float32)
        self.model = build_model(cfg, topology)
        self._sync_tensor_parallel_replicas()
        self.model = apply_fsdp2(self.model, topology)
        self.is_decoder = isinstance(self.model, MoEDecoder)
        t = cfg.training
        self.optimizer = None
        if build_optim:
            self.optimizer = build_optimizer(self.model, lr=t.learning_rate, weight_decay=t.weight_decay,
                                             betas=(0.9, 0.95), max_grad_norm=t.grad_clip, topology=topology)
        self.step_index = 0
        self.accum = max(1, t.gradient_accumulation_steps)
        self.micro = t.micro_batch_size
        self.seq = cfg.model.sequence_length
        self.stage = None
        if topology.pp_size > 1:
            self.stage = PipelineStage(topology.pp_rank, topology.pp_size, self.model, topology)
        self.last_aux: Optional[torch.Tensor] = None
        self.last_z: Optional[torch.Tensor] = None
        self.last_grad_norm: float = 0.0  # library path: global gradient norm of the last step (before clipping)

    def _sync_tensor_parallel_replicas(self) -> None:
        """Tensor-parallel ranks draw their weight slices from different random streams; everything that is NOT
        sliced (norms, router gates, embeddings under sequence parallelism, biases of row-parallel layers) must
        start identical on all of them: take the copy of the group's first rank."""
        topo = self.topology
        if topo.tp_size <= 1 or not dist.is_initialized():
            return
        from .parallel.mesh import tp_process_group

        group = tp_process_group(topo)
        src = topo.axis_ranks("tp")[0]
        with torch.no_grad():
            for p in self.model.parameters():
                if not getattr(p, "tensor_parallel_shard", False):
                    dist.broadcast(p.data, src=src, group=group)

    # ---- batch helpers --------------------------------------------------------------------------------
    @property
    def tokens_per_step_per_rank(self) -> int:
        return self.micro * self.accum * self.seq

    @property
    def tokens_per_step_global(self) -> int:
        return self.tokens_per_step_per_rank * self.topology.data_replicas

    def synthetic_batch(self, generator: Optional[torch.Generator] = None, pinned: bool = True
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Uniform-random token ids and targets of one step for this rank, on the host."""
        shape = (self.micro * self.accum, self.seq)
        V = self.cfg.model.vocab_size
        ids = torch.randint(0, V, shape, generator=generator, dtype=torch.int64)
        tgt = torch.randint(0, V, shape, generator=generator, dtype=torch.int64)
        if pinned and torch.cuda.is_available():
            ids, tgt = ids.pin_memory(), tgt.pin_memory()
        return ids, tgt

    # ---- one microbatch -------------------------------------------------------------------------------
    def _microbatch_loss(self, ids: torch.Tensor, tgt: torch.Tensor) -> torch.Tensor:
        m, t = self.cfg.model, self.cfg.training
        scale = 1.0 / (ids.numel() * self.accum)
        if self.is_decoder:
            loss = self.model.loss(ids, tgt, scale=scale)
        else:
            logits = self.model(ids)
            loss = torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), tgt.view(-1),
                                                     reduction="sum") * scale
        if (m.aux_loss_coeff > 0 or t.z_loss_weight > 0) and hasattr(self.model, "aux_losses"):
            aux, z = self.model.aux_losses()
            self.last_aux, self.last_z = aux.detach(), z.detach()
            if m.aux_loss_coeff > 0:
                loss = loss + (m.aux_loss_coeff / self.accum) * aux
            if t.z_loss_weight > 0:
                loss = loss + (t.z_loss_weight / self.accum) * z
        return loss

    # ---- one optimizer step ---------------------------------------------------------------------------
    def train_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        dev = self.device
        if ids.device != dev:
            ids = ids.to(dev, non_blocking=True)
            targets = targets.to(dev, non_blocking=True)
        lr = lr_at(self.step_index, self.cfg.training.learning_rate, self.cfg.training.warmup_steps,
                   self.cfg.training.max_steps)
        total = torch.zeros((), device=dev, dtype=torch.float32)
        if self.stage is not None:
            total = self._pipeline_step(ids, targets)
        else:
            for a in range(self.accum):
                sl = slice(a * self.micro, (a + 1) * self.micro)
                loss = self._microbatch_loss(ids[sl], targets[sl])
                loss.backward()
                total = total + loss.detach().float()
        if self.topology.tp_size > 1 and self.cfg.parallelism.sequence_parallel:
            finalize_sequence_parallel_grads(self.model, self.topology, optimizer=self.optimizer)
        if self.optimizer is not None:
            if isinstance(self.optimizer, FusedAdamW):
                self.optimizer.step(lr)
            else:
                for g in self.optimizer.param_groups:
                    g["lr"] = lr
                self._reduce_grads_library()
                if self.cfg.training.grad_clip > 0:
                    self._clip_grads_library(self.cfg.training.grad_clip)
                self.optimizer.step()
                self.optimizer.zero_grad(set_to_none=True)
        self.step_index += 1
        return total

    def _reduce_grads_library(self) -> None:
        """Average gradients over the ranks that saw different data (CPU / fp32 path with a stock optimizer):
        dense parameters over the dense-replica group (data-parallel ranks, and expert-parallel ranks too when
        expert parallelism is a mesh axis of its own), expert parameters over the replicas of the same experts;
        an expert's gradient already sums the tokens its expert-parallel group sent it."""
        topo = self.topology
        if not dist.is_initialized() or topo.data_replicas == 1:
            return
        from .parallel.mesh import ddp_process_group, edp_process_group

        ddp_group, edp_group = ddp_process_group(topo), edp_process_group(topo)
        for p in self.model.parameters():
            if p.grad is None:
                continue
            if getattr(p, "is_expert_param", False):
                if edp_group is not None:
                    dist.all_reduce(p.grad, group=edp_group)
            elif ddp_group is not None:
                dist.all_reduce(p.grad, group=ddp_group)
            p.grad.div_(topo.data_replicas)

    def _clip_grads_library(self, max_norm: float) -> None:
        """Global-norm clipping where every rank arrives at the same norm: replicated parameters count once,
        tensor-parallel slices are summed over the tensor-parallel group, expert shards over the ranks that hold
        different experts, and everything over the pipeline stages."""
        topo = self.topology
        # [replicated over tp, sliced over tp] x [dense, expert]
        sq = {(sh, ex): torch.zeros((), dtype=torch.float64, device=self.device) for sh in (0, 1) for ex in (0, 1)}
        for p in self.model.parameters():
            if p.grad is None:
                continue
            key = (int(bool(getattr(p, "tensor_parallel_shard", False)) and topo.tp_size > 1),
                   int(bool(getattr(p, "is_expert_param", False))))
            sq[key] += p.grad.detach().double().pow(2).sum()
        if dist.is_initialized() and topo.world_size > 1:
            from .parallel.mesh import ep_process_group, pp_process_group, tp_process_group

            if topo.tp_size > 1:  # slices of one matrix live on different tensor-parallel ranks
                sliced = torch.stack([sq[(1, 0)], sq[(1, 1)]])
                dist.all_reduce(sliced, group=tp_process_group(topo))
                sq[(1, 0)], sq[(1, 1)] = sliced[0], sliced[1]
            expert_sq = sq[(0, 1)] + sq[(1, 1)]
            if topo.ep_size > 1:
                dist.all_reduce(expert_sq, group=ep_process_group(topo))
            total = sq[(0, 0)] + sq[(1, 0)] + expert_sq
            if topo.pp_size > 1:
                dist.all_reduce(total, group=pp_process_group(topo))
        else:
            total = sum(sq.values())
        self.last_grad_norm = float(total.sqrt())
        coef = float(max_norm / (total.sqrt() + 1e-6))
        if coef < 1.0:
            for p in self.model.parameters():
                if p.grad is not None:
                    p.grad.mul_(coef)

    def _pipeline_step(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        m = self.cfg.parallelism.pipeline_microbatches or self.accum
        mb = ids.shape[0] // m
        mbs = [ids[i * mb:(i + 1) * mb] for i in range(m)]
        tg = [targets[i * mb:(i + 1) * mb] for i in range(m)]
        S = self.seq // (self.topology.tp_size if self.cfg.parallelism.sequence_parallel else 1)
        act_shape = (mb, S, self.cfg.model.hidden_dim)
        model = self.model
        scale = 1.0 / (mb * self.seq * m)
        coeff = self.cfg.model.aux_loss_coeff

        class _StageModule(torch.nn.Module):
            """Runs this stage; on the last stage the output is the scalar loss of the microbatch."""

            def __init__(self):
                super().__init__()
                self.calls = 0

            def forward(self, x):
                i = self.calls
                self.calls += 1
                out = model.loss(x, tg[i], scale=scale) if model.is_last_stage else model(x)
                if coeff > 0:
                    aux, _ = model.aux_losses()
                    term = aux * (coeff / m)
                    out = out + term if model.is_last_stage else _AttachAux.apply(out, term)
                return out

        stage_mod = _StageModule()
        self.stage.module = stage_mod
        outs, losses = self.stage.run_1f1b_distributed(
            mbs if model.is_first_stage else [], loss_fn=(lambda out: out) if model.is_last_stage else None,
            num_microbatches=m, activation_shape=act_shape, activation_dtype=self.dtype, device=self.device)
        total = torch.zeros((), device=self.device, dtype=torch.float32)
        for l in losses:
            total = total + l.detach().float()
        self.stage.module = self.model
        # only the last stage saw the loss: hand it to the other stages so that every rank returns (and logs) it
        from .parallel.mesh import pp_process_group

        dist.broadcast(total, src=self.topology.axis_ranks("pp")[-1], group=pp_process_group(self.topology))
        return total

    def close(self) -> None:
        pass
