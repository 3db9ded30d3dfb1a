"""``MoEDecoder``: a causal transformer whose every feed-forward is a routed mixture of SwiGLU experts.

Per block: ``x += Attention(RMSNorm(x))`` (rotary position embedding, grouped-query attention, causal) then
``x += MoE(RMSNorm(x))``.  This is the architecture the benchmark configurations name (heads, GQA, RoPE,
load-balance loss); the reference's only model has no attention (pkg/models/moe.py:148-186), so apart from
the shared ``embed`` / ``blocks[i].norm`` / ``blocks[i].moe`` / ``norm`` / ``lm_head`` attribute paths this
file has no counterpart there.

Parallelism: attention projections are column/row tensor-parallel (with Megatron sequence parallelism when
``parallelism.sequence_parallel``), experts are expert-parallel (+ tensor-parallel on the FFN width), and with
``pipeline_parallel > 1`` each rank builds only the blocks of its own stage (first stage: embedding; last
stage: final norm and LM head).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..parallel import collectives as C
from ..parallel.mesh import ParallelTopology, tp_process_group
from ..parallel.moe_layer import DistributedMoELayer
from ..parallel.pipeline_parallel import partition_layers
from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .moe import DTYPE_MAP, RMSNorm
from .registry import register_model

__all__ = ["MoEDecoder", "DecoderBlock", "CausalSelfAttention", "lm_head_loss"]


class CausalSelfAttention(nn.Module):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, rope_theta: float,
                 max_seq: int, topology: ParallelTopology, dtype: torch.dtype, sequence_parallel: bool = False):
        super().__init__()
        tp = topology.tp_size
        if num_heads % tp or num_kv_heads % tp:
            raise ValueError(f"num_heads ({num_heads}) and num_kv_heads ({num_kv_heads}) must divide by tp ({tp})")
        self.topology = topology
        self.nh, self.nkv, self.hd = num_heads // tp, num_kv_heads // tp, head_dim
        self.rope_theta, self.max_seq = rope_theta, max_seq
        self.sequence_parallel = sequence_parallel and tp > 1
        qkv_out = (num_heads + 2 * num_kv_heads) * head_dim
        self.wqkv = ColumnParallelLinear(hidden, qkv_out, bias=False, topology=topology, dtype=dtype,
                                         gather_output=False, sequence_parallel=self.sequence_parallel)
        self.wo = RowParallelLinear(num_heads * head_dim, hidden, bias=False, topology=topology, dtype=dtype,
                                    sequence_parallel=self.sequence_parallel)
        self._tables: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def _rope_tables(self, seq: int, device: torch.device):
        if self._tables is None or self._tables[0].device != device or self._tables[0].shape[0] < seq:
            self._tables = OF.rope_tables(max(seq, self.max_seq), self.hd, self.rope_theta, device)
        return self._tables

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        qkv = self.wqkv(x)  # [B, S, (nh + 2 nkv) * hd] with the full sequence
        B, S, _ = qkv.shape
        heads = self.nh + 2 * self.nkv
        cos, sin = self._rope_tables(S, qkv.device)
        o = OF.rope_causal_attention(qkv.view(B, S, heads, self.hd), cos, sin, self.nh, self.nkv)
        return self.wo(o.reshape(B, S, self.nh * self.hd))


class DecoderBlock(nn.Module):
    def __init__(self, cfg, topology: ParallelTopology, dtype: torch.dtype):
        super().__init__()
        m, par = cfg.model, cfg.parallelism
        sp = bool(par.sequence_parallel) and topology.tp_size > 1
        self.sequence_parallel = sp
        self.topology = topology
        self.attn_norm = RMSNorm(m.hidden_dim, eps=m.norm_eps, dtype=dtype)
        self.attn = CausalSelfAttention(m.hidden_dim, m.resolved_num_heads, m.resolved_num_kv_heads,
                                        m.resolved_head_dim, m.rope_theta, m.sequence_length, topology, dtype, sp)
        self.norm = RMSNorm(m.hidden_dim, eps=m.norm_eps, dtype=dtype)
        self.moe = DistributedMoELayer(m.hidden_dim, m.ffn_dim, m.num_experts, m.top_k, topology,
                                       capacity_factor=m.capacity_factor, capacity_dropping=m.capacity_dropping,
                                       dtype=dtype, init_std=(m.init_std if m.init_std > 0 else None))
        if sp:
            for p in list(self.attn_norm.parameters()) + list(self.norm.parameters()):
                p.sequence_parallel_grad = True  # partial per TP rank: summed over the TP group after backward
            if self.moe.fused_sequence_shard_path(self.moe.w13):
                # the layer will take sequence shards: its router then sees a shard only (known now, so that the
                # optimizer can group the gate with the other partially summed parameters)
                self.moe.router.gate_w.sequence_parallel_grad = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.attn_norm(x))
        h = self.norm(x)
        if self.sequence_parallel and self.moe.fused_sequence_shard_path(h):
            # peer-memory path: the layer takes the shard; the sequence gather is the row pull inside its first
            # grouped GEMM, the reduce-scatter the row push of its second one
            y = self.moe(h, sequence_shard=True)
        elif self.sequence_parallel:
            group = tp_process_group(self.topology)
            full = C.all_gather(h, 1, group, reduce_scatter_grad=False)
            y = self.moe(full)  # replicated result (the layer all-reduces over TP)
            y = C.split(y, 1, group)
        else:
            y = self.moe(h)
        return x + y


class _LMHeadLossFn(torch.autograd.Function):
    """sum-CE(h @ W^T, targets) * scale without keeping the logits: per chunk of rows one tcgen05 GEMM for the
    logits, the cross-entropy kernel (loss sum, logits overwritten by their gradient), and - only when a gradient
    will be asked for - the two gradient GEMMs (``dh`` with W read N-major, ``dW`` added into an fp32 buffer by the
    TMA reduce-add epilogue).  ``backward`` scales both by the incoming gradient; ``dW`` goes to ``W.main_grad``
    when the optimizer gave the weight one."""

    @staticmethod
    def forward(ctx, h, weight, targets, scale, chunk):
        from ..ops import _ext, kernels

        ext = _ext.ext()
        N = h.shape[0]
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        loss = torch.zeros(1, device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.empty(weight.shape, device=h.device, dtype=torch.float32) if need_dw else None
        for a in range(0, N, chunk):
            b = min(a + chunk, N)
            logits = kernels.linear_nt(h[a:b], weight)
            ext.cross_entropy(logits, targets[a:b], loss, scale)  # logits now hold d(loss)/d(logits)
            if need_dh:
                kernels.linear_nn(logits, weight, out=dh[a:b])
            if need_dw:
                kernels.linear_tn_acc(logits, h[a:b], dw, accumulate=a > 0)
        ctx.save_for_backward(dh, dw, weight)
        return loss[0] * scale

    @staticmethod
    def backward(ctx, g):
        dh, dw, weight = ctx.saved_tensors
        if dh is not None:
            dh = dh * g.to(dh.dtype)
        if dw is not None:
            main = getattr(weight, "main_grad", None)
            if main is not None:
                main.addcmul_(dw, g.to(torch.float32))
                dw = None
            else:
                dw = (dw * g.to(torch.float32)).to(weight.dtype)
        return dh, dw, None, None, None


def lm_head_loss(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, scale: float, chunk: int = 4096
                 ) -> torch.Tensor:
    """``scale * sum_t CE(h_t @ W^T, target_t)``; h [N, H], weight [V, H], targets [N] (negative = ignored)."""
    if OF.linear_supported(h, weight):
        return _LMHeadLossFn.apply(OF.rows_for_tma(h), weight, targets.contiguous(), scale, chunk)
    logits = F.linear(h, weight).float()
    return F.cross_entropy(logits, targets, reduction="sum", ignore_index=-100) * scale


@register_model("moe_decoder")
class MoEDecoder(nn.Module):
    def __init__(self, cfg, topology: ParallelTopology):
        super().__init__()
        m = cfg.model
        dtype = DTYPE_MAP.get(m.dtype, torch.float32)
        self.cfg, self.topology, self.dtype = cfg, topology, dtype
        self.num_layers_total = m.num_layers
        self.stage_layers = list(partition_layers(m.num_layers, topology.pp_size)[topology.pp_rank])
        self.is_first_stage, self.is_last_stage = topology.is_first_pp_stage(), topology.is_last_pp_stage()
        self.sequence_parallel = bool(cfg.parallelism.sequence_parallel) and topology.tp_size > 1
        self.embed = nn.Embedding(m.vocab_size, m.hidden_dim, dtype=dtype) if self.is_first_stage else None
        self.blocks = nn.ModuleList([DecoderBlock(cfg, topology, dtype) for _ in self.stage_layers])
        self.norm = RMSNorm(m.hidden_dim, eps=m.norm_eps, dtype=dtype) if self.is_last_stage else None
        self.lm_head = nn.Linear(m.hidden_dim, m.vocab_size, bias=False, dtype=dtype) if self.is_last_stage else None
        if m.init_std > 0:
            self._init_weights(m.init_std)
        if self.sequence_parallel:
            for mod in (self.embed, self.norm, self.lm_head):
                if mod is not None:
                    for p in mod.parameters():
                        p.sequence_parallel_grad = True
        from ..parallel.data_parallel import mark_expert_params

        mark_expert_params(self)

    def _init_weights(self, std: float) -> None:
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, mean=0.0, std=std)

    # ---- pieces used by the pipeline schedule and the trainer ---------------------------------------
    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.embed(ids)
        if self.sequence_parallel:
            x = C.split(x, 1, tp_process_group(self.topology))
        return x

    def run_blocks(self, x: torch.Tensor) -> torch.Tensor:
        recompute = bool(self.cfg.training.activation_recompute) and torch.is_grad_enabled()
        for blk in self.blocks:
            if recompute:
                from torch.utils.checkpoint import checkpoint

                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x = blk(x)
        return x

    def final_hidden(self, x: torch.Tensor) -> torch.Tensor:
        return self.norm(x)

    def forward(self, ids_or_hidden: torch.Tensor) -> torch.Tensor:
        """Stage forward.  First stage takes token ids [B, S]; the last stage returns logits [B, S, V]."""
        x = self.embed_tokens(ids_or_hidden) if self.is_first_stage else ids_or_hidden
        x = self.run_blocks(x)
        if not self.is_last_stage:
            return x
        x = self.final_hidden(x)
        if self.sequence_parallel:
            x = C.all_gather(x, 1, tp_process_group(self.topology), reduce_scatter_grad=False)
        return OF.linear(x, self.lm_head.weight)

    def loss(self, ids_or_hidden: torch.Tensor, targets: torch.Tensor, scale: Optional[float] = None
             ) -> torch.Tensor:
        """Cross-entropy of the next-token targets [B, S] (mean over tokens unless ``scale`` is given), computed
        without materialising the [B*S, V] logits on the device path.  Last stage only."""
        x = self.embed_tokens(ids_or_hidden) if self.is_first_stage else ids_or_hidden
        x = self.final_hidden(self.run_blocks(x))
        tgt = targets
        if self.sequence_parallel:
            tp, r = self.topology.tp_size, self.topology.tp_rank
            tgt = targets.chunk(tp, dim=1)[r]
        n = tgt.numel()
        if scale is None:
            scale = 1.0 / max(targets.numel(), 1)
        loss = lm_head_loss(x.reshape(n, -1), self.lm_head.weight, tgt.reshape(-1), scale)
        if self.sequence_parallel:
            loss = C.all_reduce(loss, tp_process_group(self.topology))
        return loss

    def moe_layers(self) -> List[DistributedMoELayer]:
        return [blk.moe for blk in self.blocks]

    def aux_losses(self) -> Tuple[torch.Tensor, torch.Tensor]:
        aux = [l.router.last_aux_loss * l.aux_scale for l in self.moe_layers() if l.router.last_aux_loss is not None]
        z = [l.router.last_z_loss * l.aux_scale for l in self.moe_layers() if l.router.last_z_loss is not None]
        dev = next(self.parameters()).device
        zero = torch.zeros((), device=dev, dtype=torch.float32)
        n = max(self.num_layers_total, 1)
        a = torch.stack(aux).sum() / n if aux else zero
        zl = torch.stack(z).sum() / n if z else zero
        if any(l.aux_scale != 1.0 for l in self.moe_layers()):
            # the routers saw sequence shards: each rank holds its shard's share of the two terms.  Sum them over the
            # tensor-parallel group so that every rank reports the same value; the backward of this sum is the
            # identity, so each rank still back-propagates its own share only
            both = C.all_reduce(torch.stack([a, zl]), tp_process_group(self.topology))
            a, zl = both[0], both[1]
        return a, zl

    def count_parameters(self) -> Dict[str, int]:
        total = sum(p.numel() for p in self.parameters())
        embed = sum(p.numel() for mod in (self.embed, self.lm_head) if mod is not None for p in mod.parameters())
        router = sum(p.numel() for l in self.moe_layers() for p in l.router.parameters())
        experts = sum(l.w13.numel() + l.w2.numel() for l in self.moe_layers())
        attn = sum(p.numel() for blk in self.blocks for p in blk.attn.parameters())
        return {"total": total, "embed": embed, "moe_router": router, "moe_experts": experts, "attention": attn,
                "other": total - embed - router - experts - attn}


def finalize_sequence_parallel_grads(model: nn.Module, topology: ParallelTopology, optimizer=None) -> None:
    """Sum over the TP group the gradients of parameters that saw only this rank's sequence shard.  The fused
    optimizer keeps those gradients at the front of one flat buffer and sums them with one collective; whatever it
    does not cover (another optimizer, a parameter flagged after the optimizer was built) is summed one by one."""
    import torch.distributed as dist

    if topology.tp_size == 1 or not dist.is_initialized():
        return
    group = tp_process_group(topology)
    done = set()
    if optimizer is not None and hasattr(optimizer, "allreduce_sequence_parallel_grads"):
        done = optimizer.allreduce_sequence_parallel_grads(group)
    for p in model.parameters():
        if not getattr(p, "sequence_parallel_grad", False) or id(p) in done:
            continue
        main = getattr(p, "main_grad", None)
        if main is not None:  # fused optimizer: kernel-accumulated and autograd parts meet in the fp32 buffer
            if p.grad is not None:
                main.add_(p.grad)
                p.grad = None
            dist.all_reduce(main, group=group)
        elif p.grad is not None:
            dist.all_reduce(p.grad, group=group)
