"""Pipeline parallelism: one ``PipelineStage`` per rank of the pipeline axis, 1F1B schedule.

API of the reference stage (pkg/distributed/pipeline_parallel.py:52-374): ``PipelineStage(stage_id,
num_stages, module=None, topology=None)``, ``is_first`` / ``is_last``, ``forward_step``, ``backward_step``,
``run_1f1b`` (single-process schedule check) and ``run_1f1b_distributed(micro_batches, loss_fn)``.

Transport stays on the library point-to-point path (NCCL on GPUs, gloo on CPU).  Differences from the
reference: a send towards a neighbour and the receive from the same neighbour are posted together with
``batch_isend_irecv`` (separate blocking ``send``/``recv`` calls in opposite order deadlock on NCCL and the
reference's CPU ``int64[2]`` header tensor is not accepted by NCCL at all, ``pipeline_parallel.py:131,151``);
the activation shape is an explicit argument (or taken from the first microbatch) rather than a header;
neighbours are looked up through the topology instead of ``rank -/+ ep_size``; warm-up depth is
``num_stages - stage_id - 1`` so every stage runs the same number of forwards and backwards.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .mesh import ParallelTopology, pp_process_group

__all__ = ["PipelineStage", "partition_layers"]


def partition_layers(num_layers: int, num_stages: int) -> List[range]:
    """Contiguous, balanced layer ranges; earlier stages take the remainder."""
    per, rem = divmod(num_layers, num_stages)
    out, start = [], 0
    for s in range(num_stages):
        n = per + (1 if s < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


class PipelineStage:
    def __init__(self, stage_id: int, num_stages: int, module: Optional[nn.Module] = None,
                 topology: Optional[ParallelTopology] = None):
        if stage_id < 0 or stage_id >= num_stages:
            raise ValueError(f"stage_id ({stage_id}) must be in [0, num_stages={num_stages})")
        self.stage_id, self.num_stages = int(stage_id), int(num_stages)
        self.module = module
        self.topology = topology
        self._multi_process = topology is not None and topology.pp_size > 1 and dist.is_initialized()
        self._pp_group = pp_process_group(topology) if self._multi_process else None
        self._activation_stash: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._sends_in_flight: List[Tuple[list, list]] = []

    # ---- position -----------------------------------------------------------------------------
    @property
    def is_first(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last(self) -> bool:
        return self.stage_id == self.num_stages - 1

    def _neighbour(self, delta: int) -> Optional[int]:
        if self.topology is None:
            return None
        s = self.stage_id + delta
        if s < 0 or s >= self.num_stages:
            return None
        return self.topology.axis_ranks("pp")[s]

    def _prev_rank(self) -> Optional[int]:
        return self._neighbour(-1)

    def _next_rank(self) -> Optional[int]:
        return self._neighbour(+1)

    # ---- transport ----------------------------------------------------------------------------
    def _exchange(self, send_prev=None, send_next=None, recv_prev=None, recv_next=None) -> None:
        """Post all given sends / receives as one batch.  A batch that receives something is waited for at once
        (the caller needs the data next); a batch of sends only is left in flight and collected at the next
        exchange, so the compute stream does not stall on a neighbour that has not posted its receive yet and the
        transfer overlaps the compute that follows.  The sent tensors stay referenced until then."""
        ops, keep = [], []
        if send_prev is not None:
            t = send_prev.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self._prev_rank()))
        if recv_prev is not None:
            ops.append(dist.P2POp(dist.irecv, recv_prev, self._prev_rank()))
        if send_next is not None:
            t = send_next.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self._next_rank()))
        if recv_next is not None:
            ops.append(dist.P2POp(dist.irecv, recv_next, self._next_rank()))
        if not ops:
            return
        self._collect_sends()
        reqs = dist.batch_isend_irecv(ops)
        if recv_prev is None and recv_next is None:
            self._sends_in_flight.append((reqs, keep))
            return
        for req in reqs:
            req.wait()

    def _collect_sends(self) -> None:
        pending, self._sends_in_flight = self._sends_in_flight, []
        for reqs, _keep in pending:
            for req in reqs:
                req.wait()

    _HEADER_DTYPES = (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32)
    _HEADER_LEN = 12  # count, dtype code, rank, up to 9 extents

    def _send_header(self, m: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> None:
        if len(shape) > self._HEADER_LEN - 3:
            raise ValueError(f"activation rank {len(shape)} does not fit the pipeline header")
        vals = [m, self._HEADER_DTYPES.index(dtype), len(shape), *shape]
        vals += [0] * (self._HEADER_LEN - len(vals))
        self._exchange(send_next=torch.tensor(vals, dtype=torch.int64, device=device))

    def _recv_header(self, device: torch.device) -> Tuple[int, Tuple[int, ...], torch.dtype]:
        """Receive the header from the previous stage and pass a zero-count header on at once (the real one for the
        next stage follows this stage's first forward, when the shape of its output is known)."""
        buf = torch.empty(self._HEADER_LEN, dtype=torch.int64, device=device)
        self._exchange(recv_prev=buf)
        vals = buf.tolist()
        m, code, nd = int(vals[0]), int(vals[1]), int(vals[2])
        if m == 0 and not self.is_last:
            self._send_header(0, (), torch.float32, device)
        return m, tuple(int(v) for v in vals[3: 3 + nd]), self._HEADER_DTYPES[code]

    # ---- single steps -------------------------------------------------------------------------
    def forward_step(self, micro_batch: torch.Tensor) -> torch.Tensor:
        """Apply this stage's module (in a multi-process pipeline: receive, apply, send)."""
        if self._multi_process:
            x = micro_batch
            if not self.is_first:
                x = torch.empty_like(micro_batch)
                self._exchange(recv_prev=x)
            out = self.module(x) if self.module is not None else x
            if not self.is_last:
                self._exchange(send_next=out.detach())
                self._collect_sends()
            return out
        return self.module(micro_batch) if self.module is not None else micro_batch

    def backward_step(self, grad_output: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Pass-through: the distributed backward lives inside :meth:`run_1f1b_distributed`."""
        return grad_output

    # ---- schedule check in one process -----------------------------------------------------------
    def run_1f1b(self, micro_batches: Sequence[torch.Tensor]) -> List[Optional[torch.Tensor]]:
        """Walk the warm-up / steady / drain phases locally; returns one gradient stand-in per microbatch."""
        p, m = self.num_stages, len(micro_batches)
        acts: List[Optional[torch.Tensor]] = [None] * m
        grads: List[Optional[torch.Tensor]] = [None] * m
        warm = min(p - 1, m)
        for t in range(warm):
            acts[t] = self.forward_step(micro_batches[t])
        for t in range(m - warm):
            acts[t + warm] = self.forward_step(micro_batches[t + warm])
            grads[t] = self.backward_step(torch.ones_like(acts[t]))
        for t in range(m - warm, m):
            grads[t] = self.backward_step(torch.ones_like(acts[t]))
        return grads

    # ---- the real thing -----------------------------------------------------------------------
    def run_1f1b_distributed(
        self,
        micro_batches: Sequence[torch.Tensor],
        loss_fn: Optional[Callable[..., torch.Tensor]] = None,
        num_microbatches: Optional[int] = None,
        activation_shape: Optional[Sequence[int]] = None,
        activation_dtype: Optional[torch.dtype] = None,
        device: Optional[torch.device] = None,
    ) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
        """Run ``m`` microbatches through this stage with the 1F1B schedule.

        First stage: ``micro_batches`` are the inputs.  Other stages receive activations of
        ``activation_shape`` / ``activation_dtype`` (default: shape and dtype of ``micro_batches[0]``).
        Last stage: ``loss_fn(output)`` or ``loss_fn(output, mb_index)`` gives the scalar to back-propagate
        (default ``output.sum()``).  Returns ``(outputs, losses)``; both are only filled on the last stage.
        """
        if not self._multi_process:
            raise RuntimeError("run_1f1b_distributed requires pp_size > 1 and dist.is_initialized(). "
                               "Use run_1f1b() for single-process scheduling.")
        # Callers that give neither a count nor a shape use the reference's convention
        # (pkg/distributed/pipeline_parallel.py:126-179): only the first stage holds micro-batches, later stages pass
        # an empty list and learn the count, shape and dtype from a small header that travels down the pipeline ahead
        # of the first activation.  All stages of one call must use the same convention.
        announce = num_microbatches is None and activation_shape is None
        device = device or (self.topology.device if self.topology is not None else torch.device("cpu"))
        if announce and not self.is_first:
            m, activation_shape, activation_dtype = self._recv_header(device)
        else:
            m = num_microbatches if num_microbatches is not None else len(micro_batches)
        if m == 0:
            if announce and self.is_first and not self.is_last:
                self._send_header(0, (), torch.float32, device)
            self._collect_sends()
            return [], []
        if not self.is_first:
            if activation_shape is None:
                if not micro_batches:
                    raise ValueError("non-first stages need activation_shape or a template microbatch")
                activation_shape = tuple(micro_batches[0].shape)
                activation_dtype = activation_dtype or micro_batches[0].dtype
                device = micro_batches[0].device
            activation_dtype = activation_dtype or torch.float32

        import inspect

        two_arg_loss = loss_fn is not None and len(inspect.signature(loss_fn).parameters) >= 2
        inputs: Dict[int, torch.Tensor] = {}
        outs: Dict[int, torch.Tensor] = {}
        outputs: List[torch.Tensor] = []
        losses: List[torch.Tensor] = []

        def new_act():
            return torch.empty(tuple(activation_shape), dtype=activation_dtype, device=device)

        def fwd(mb: int, x: Optional[torch.Tensor]) -> torch.Tensor:
            if self.is_first:
                x = micro_batches[mb]
            if x.is_floating_point():
                x = x.detach().requires_grad_(True)
            out = self.module(x) if self.module is not None else x
            inputs[mb], outs[mb] = x, out
            if self.is_last:
                loss = (loss_fn(out, mb) if two_arg_loss else loss_fn(out)) if loss_fn is not None else out.sum()
                outputs.append(out.detach())
                losses.append(loss)
                outs[mb] = loss
            return out

        def bwd(mb: int, grad: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
            x, out = inputs.pop(mb), outs.pop(mb)
            if self.is_last:
                out.backward()
            else:
                out.backward(grad)
            return x.grad if (x.is_floating_point() and not self.is_first) else None

        warm = min(self.num_stages - self.stage_id - 1, m)
        steady = m - warm
        recv_buf: Optional[torch.Tensor] = None
        # first activation
        if not self.is_first:
            recv_buf = new_act()
            self._exchange(recv_prev=recv_buf)
        # warm-up forwards
        for i in range(warm):
            out = fwd(i, recv_buf)
            if announce and i == 0 and not self.is_last:
                self._send_header(m, tuple(out.shape), out.dtype, device)
            nxt = None
            if not self.is_first and (i + 1 < m):
                nxt = new_act()
            self._exchange(send_next=None if self.is_last else out.detach(), recv_prev=nxt)
            recv_buf = nxt
        # steady state: one forward, one backward
        grad_buf: Optional[torch.Tensor] = None
        for i in range(steady):
            f_mb, b_mb = warm + i, i
            out = fwd(f_mb, recv_buf)
            if not self.is_last:
                grad_buf = torch.empty_like(out)
                self._exchange(send_next=out.detach(), recv_next=grad_buf)
            gin = bwd(b_mb, grad_buf)
            nxt = None
            if not self.is_first and (f_mb + 1 < m):
                nxt = new_act()
            self._exchange(send_prev=gin, recv_prev=nxt)
            recv_buf = nxt
        # drain backwards
        for i in range(steady, m):
            if not self.is_last:
                template = outs[i]
                grad_buf = torch.empty_like(template)
                self._exchange(recv_next=grad_buf)
            gin = bwd(i, grad_buf)
            self._exchange(send_prev=gin)
        self._collect_sends()
        return outputs, losses
