"""Fused AdamW over flat parameter buffers, with global-norm clipping and optional optimizer-state sharding.

The reference trains with ``torch.optim.AdamW(betas=(0.9, 0.95))`` + ``clip_grad_norm_`` on FSDP2-wrapped
parameters (train.py:207-212, 322-323; pkg/distributed/data_parallel.py:40-98: bf16 compute parameters,
fp32 reduction).  Here the same mixed-precision contract (bf16 parameters in the model, fp32 master copy and
moments in the optimizer) is one kernel launch per parameter group:

* parameters are re-pointed into one flat bf16 buffer per group, gradients into one flat buffer
  (fp32 ``main_grad``: the GEMM kernels add the weight gradients of experts, projections and LM head into it
  directly; what autograd leaves in ``p.grad`` - norm weights, router gates, embedding - is added at step time);
* the global gradient norm is a device scalar (sum-of-squares kernel), so clipping needs no host round trip;
* with data parallelism the flat gradient is reduce-scattered, the update runs on this rank's shard only, and
  the updated bf16 parameters are all-gathered (ZeRO-style sharding of master weights and moments).  Expert
  parameters are reduced over the ranks that hold the same experts only.

``build_optimizer`` returns ``torch.optim.AdamW`` for CPU / fp32 models (the reference behaviour).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _ext


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _FlatGroup:
    """One flat bf16 parameter buffer + gradient buffer + (sharded) fp32 master / moments."""

    def __init__(self, name: str, params: List[nn.Parameter], grad_dtype: torch.dtype, weight_decay_mask: List[bool],
                 shard_group=None, topology=None, axis: str = "dp", param_names: Optional[List[str]] = None):
        self.name, self.params = name, params
        self.param_names = list(param_names) if param_names is not None else [f"{name}.{i}" for i in range(len(params))]
        dev = params[0].device
        self.shard_group = shard_group
        self.shard_world = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.shard_rank = dist.get_rank(shard_group) if shard_group is not None else 0
        offs, total = [], 0
        for p in params:
            offs.append(total)
            total += _align(p.numel(), 8)
        self.numel = _align(total, 8 * 16 * self.shard_world)
        self.offsets = offs
        self.peer = None
        if self.shard_world > 1:
            from ..parallel import symm_dp

            self.peer = symm_dp.make_peer(topology, axis, name, self.numel, grad_dtype)
        if self.peer is not None:  # buffers in symmetric memory: peers reduce / push straight from them
            self.flat_p, self.flat_g = self.peer.flat_p, self.peer.flat_g
        else:
            self.flat_p = torch.zeros(self.numel, device=dev, dtype=torch.bfloat16)
            self.flat_g = torch.zeros(self.numel, device=dev, dtype=grad_dtype)
        self.decay = weight_decay_mask
        # parameters that every tensor-parallel rank holds whole (norms, router gates, embeddings under sequence
        # parallelism): their squared gradient norm must count once, not once per tensor-parallel rank
        tp = topology.tp_size if topology is not None else 1
        self.tp_size = tp
        self.replicated = [tp > 1 and not getattr(p, "tensor_parallel_shard", False) for p in params]
        # leading run of parameters whose gradients are partial sums over the tensor-parallel group (they saw a
        # sequence shard): build_optimizer puts them first, so one all-reduce over flat_g[:sp_prefix] sums them all
        self.sp_prefix = 0
        self.sp_prefix_ids = set()
        for p, off in zip(params, offs):
            if not getattr(p, "sequence_parallel_grad", False):
                break
            self.sp_prefix = off + _align(p.numel(), 8)
            self.sp_prefix_ids.add(id(p))
        for p, off in zip(params, offs):
            n = p.numel()
            self.flat_p[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_p[off:off + n].view(p.shape)
            gview = self.flat_g[off:off + n].view(p.shape)
            if grad_dtype == torch.float32:
                p.main_grad = gview
                p.grad = None
            else:
                p.grad = gview
        self.shard_numel = self.numel // self.shard_world
        lo = self.shard_rank * self.shard_numel
        self.shard_lo = lo
        self.master = self.flat_p[lo:lo + self.shard_numel].float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        # per-element decay is applied per segment: split the shard into decay / no-decay runs
        self._segments = self._build_segments()
        self.grad_scale = 1.0  # extra factor on this group's gradients (1/ep for expert weights, see build_optimizer)

    def _build_segments(self) -> List[Tuple[int, int, bool, bool]]:
        """(start, end, decay, replicated over tp) runs inside this rank's shard, in shard-local coordinates."""
        segs: List[Tuple[int, int, bool, bool]] = []
        lo, hi = self.shard_lo, self.shard_lo + self.shard_numel
        bounds = self.offsets + [self.numel]
        for i, (d, r) in enumerate(zip(self.decay, self.replicated)):
            a, b = max(bounds[i], lo), min(bounds[i + 1], hi)
            if a >= b:
                continue
            if segs and segs[-1][2] == d and segs[-1][3] == r and segs[-1][1] == a - lo:
                segs[-1] = (segs[-1][0], b - lo, d, r)
            else:
                segs.append((a - lo, b - lo, d, r))
        return segs

    def reassign_grads(self) -> None:
        """Bring gradients that autograd left in ``p.grad`` into the flat buffer.  fp32 groups: added to
        ``main_grad`` (where the GEMM kernels already accumulated the matrix gradients) and dropped; bf16 groups:
        ``p.grad`` is pointed back at its slice of the flat buffer."""
        if self.flat_g.dtype == torch.float32:
            for p in self.params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad)
                    p.grad = None
            return
        for p, off in zip(self.params, self.offsets):
            view = self.flat_g[off:off + p.numel()].view(p.shape)
            if p.grad is None:
                p.grad = view
            elif p.grad.data_ptr() != view.data_ptr():
                view.add_(p.grad.to(view.dtype))
                p.grad = view


class FusedAdamW:
    """AdamW (decoupled decay) on flat buffers; one ``adamw`` kernel launch per decay run of each group."""

    def __init__(self, groups: List[_FlatGroup], lr: float, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 0.0, norm_groups: Iterable = ()):
        self.groups = groups
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        dev = groups[0].flat_p.device
        self.sumsq = torch.zeros(1, device=dev, dtype=torch.float32)
        self._tmp = torch.zeros(1, device=dev, dtype=torch.float32)
        self.last_grad_norm_sq: Optional[torch.Tensor] = None
        self._norm_groups = list(norm_groups)  # process groups over which the squared norm is summed
        self.param_groups = [{"lr": lr, "params": [p for g in groups for p in g.params]}]
        self._pre_step_hooks: List = []

    def register_step_pre_hook(self, hook) -> None:
        """``hook(optimizer, args, kwargs)`` runs at the start of every ``step`` (the ``torch.optim.Optimizer``
        name and signature).  The asynchronous checkpointer uses it to make the step wait for a snapshot that is
        still being copied off the device."""
        self._pre_step_hooks.append(hook)

    # -- torch.optim-like surface ----------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = False) -> None:
        for g in self.groups:
            g.flat_g.zero_()

    def state_dict(self) -> Dict:
        return {
            "step": self.step_count,
            # ``layout`` (parameter name, offset in the flat buffer, element count, shape) lets a loader that runs
            # under another sharding find any parameter's master weights and moments again
            "groups": {g.name: {"master": g.master, "m": g.m, "v": g.v, "shard_rank": g.shard_rank,
                                "shard_world": g.shard_world, "numel": g.numel, "shard_lo": g.shard_lo,
                                "layout": [(n, off, p.numel(), tuple(p.shape))
                                           for n, off, p in zip(g.param_names, g.offsets, g.params)]}
                       for g in self.groups},
            "param_groups": [{"lr": self.lr, "betas": self.betas, "eps": self.eps,
                              "weight_decay": self.weight_decay}],
            "state": {},
        }

    def load_state_dict(self, sd: Dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for g in self.groups:
            src = sd["groups"].get(g.name)
            if src is None:
                continue
            for name in ("master", "m", "v"):
                getattr(g, name).copy_(src[name].to(getattr(g, name).device))
            self._publish_params(g)

    def load_resharded(self, fetch, step: int) -> None:
        """Fill this rank's shards of master weights and moments from state written under another sharding.
        ``fetch(group_name, param_name, lo, hi)`` returns ``{"master", "m", "v"}`` for elements [lo, hi) of that
        parameter as this rank's model holds it now (flattened), or ``None`` when the old state has no such parameter."""
        self.step_count = int(step)
        for g in self.groups:
            lo_s, hi_s = g.shard_lo, g.shard_lo + g.shard_numel
            for name, off, p in zip(g.param_names, g.offsets, g.params):
                a, b = max(off, lo_s), min(off + p.numel(), hi_s)
                if a >= b:
                    continue
                src = fetch(g.name, name, a - off, b - off)
                if src is None:
                    continue
                for key in ("master", "m", "v"):
                    getattr(g, key)[a - lo_s:b - lo_s].copy_(src[key].to(g.master.device))

    # -- step ------------------------------------------------------------------------------------
    def _reduce_grads(self, g: _FlatGroup) -> torch.Tensor:
        """Returns this rank's gradient shard (averaged over the shard group)."""
        if g.shard_world == 1:
            return g.flat_g
        from ..parallel import symm_dp

        return symm_dp.reduce_scatter_grads(g)

    def _publish_params(self, g: _FlatGroup) -> None:
        """After an update of the shard: make every rank's flat bf16 parameter buffer whole again."""
        if g.shard_world == 1:
            return
        from ..parallel import symm_dp

        symm_dp.all_gather_params(g)

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> None:
        ext = _ext.ext()
        for hook in self._pre_step_hooks:
            hook(self, (), {})
        if lr is not None:
            self.lr = lr
            self.param_groups[0]["lr"] = lr
        self.step_count += 1
        shards = []
        self.sumsq.zero_()
        tmp = self._tmp
        for g in self.groups:
            g.reassign_grads()
            gs = self._reduce_grads(g)
            shards.append(gs)
            if self.max_grad_norm > 0:
                if g.tp_size > 1 and any(g.replicated):
                    # every tensor-parallel rank adds its shard to the world-wide sum: what all of them hold whole
                    # enters with weight 1/tp so that it counts once (as the library path's clipping does)
                    for a, b, _decay, rep in g._segments:
                        tmp.zero_()
                        ext.sumsq(gs[a:b], tmp)
                        self.sumsq.add_(tmp, alpha=g.grad_scale ** 2 / (g.tp_size if rep else 1))
                else:
                    tmp.zero_()
                    ext.sumsq(gs, tmp)
                    self.sumsq.add_(tmp, alpha=g.grad_scale ** 2)
        if self.max_grad_norm > 0:
            for pg in self._norm_groups:
                if pg is not None:
                    dist.all_reduce(self.sumsq, group=pg)
        self.last_grad_norm_sq = self.sumsq.clone() if self.max_grad_norm > 0 else None
        b1, b2 = self.betas
        for g, gs in zip(self.groups, shards):
            sharded = g.shard_world > 1
            p16_base = g.flat_p[g.shard_lo:g.shard_lo + g.shard_numel]
            for a, b, decay, _rep in g._segments:
                ext.adamw(g.master[a:b], p16_base[a:b], g.m[a:b], g.v[a:b], gs[a:b], self.lr, b1, b2, self.eps,
                          self.weight_decay if decay else 0.0, self.step_count, g.grad_scale, self.max_grad_norm,
                          self.sumsq if self.max_grad_norm > 0 else None, not sharded)
            if sharded:
                g.flat_g.zero_()
                self._publish_params(g)

    def allreduce_sequence_parallel_grads(self, group) -> set:
        """Sum over the tensor-parallel ``group`` the gradients of the parameters that saw only this rank's sequence
        shard, in one collective per flat group (they sit at the front of the fp32 gradient buffer).  Returns the ids
        of the parameters that were covered; anything flagged later is left to the caller."""
        done: set = set()
        for g in self.groups:
            if g.sp_prefix > 0 and g.flat_g.dtype == torch.float32:
                g.reassign_grads()  # fold what autograd left in p.grad into the buffer first
                dist.all_reduce(g.flat_g[:g.sp_prefix], group=group)
                done |= g.sp_prefix_ids
        return done

    def grad_norm(self) -> float:
        """Global gradient norm of the last step (one device read)."""
        return float(self.last_grad_norm_sq.sqrt()) if self.last_grad_norm_sq is not None else 0.0


def _no_decay(name: str, p: nn.Parameter) -> bool:
    return p.dim() <= 1 or name.endswith(".bias") or "norm" in name.lower()


def build_optimizer(model: nn.Module, lr: float, weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8,
                    max_grad_norm: float = 0.0, topology=None):
    """FusedAdamW for CUDA bf16 models, ``torch.optim.AdamW`` otherwise."""
    params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    from .functional import force_library

    on_device = all(p.is_cuda and p.dtype == torch.bfloat16 for _, p in params) and not force_library()
    if not on_device:
        decay = [p for n, p in params if not _no_decay(n, p)]
        no_decay = [p for n, p in params if _no_decay(n, p)]
        return torch.optim.AdamW(
            [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
            lr=lr, betas=betas, eps=eps)

    from ..parallel.mesh import ddp_process_group, edp_process_group

    expert = [(n, p) for n, p in params if getattr(p, "is_expert_param", False)]
    dense = [(n, p) for n, p in params if not getattr(p, "is_expert_param", False)]
    dp_group = expert_dp_group = None
    if topology is not None and dist.is_initialized() and topology.world_size > 1:
        dp_group = ddp_process_group(topology)  # None when the group has one rank
        expert_dp_group = edp_process_group(topology)
    groups: List[_FlatGroup] = []
    # parameters whose gradients need the tensor-parallel sum go first (stable: the rest keeps its order)
    dense.sort(key=lambda np_: 0 if getattr(np_[1], "sequence_parallel_grad", False) else 1)
    if dense:
        # fp32 gradient buffer: the weight-gradient GEMMs of the projections and of the LM head add into it with
        # TMA reduce-add across microbatches; vector parameters' autograd gradients are added at step time
        groups.append(_FlatGroup("dense", [p for _, p in dense], torch.float32,
                                 [not _no_decay(n, p) for n, p in dense], shard_group=dp_group, topology=topology,
                                 axis="ddp", param_names=[n for n, _ in dense]))
    if expert:
        groups.append(_FlatGroup("expert", [p for _, p in expert], torch.float32, [True] * len(expert),
                                 shard_group=expert_dp_group, topology=topology, axis="edp",
                                 param_names=[n for n, _ in expert]))
        # an expert's gradient already sums the contributions of the `ep` ranks whose tokens it served; the
        # objective is the mean over all data-parallel ranks, so 1/ep is still missing after the edp average
        if topology is not None and dist.is_initialized() and topology.ep_size > 1:
            groups[-1].grad_scale = 1.0 / topology.ep_size
    norm_groups = []
    if topology is not None and dist.is_initialized() and topology.world_size > 1:
        norm_groups = [dist.group.WORLD]
    return FusedAdamW(groups, lr, betas, eps, weight_decay, max_grad_norm, norm_groups)
