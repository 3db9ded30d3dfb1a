"""Headline benchmark: MoE training throughput (tokens/s, MFU) on the OLMoE-1B-7B-shaped configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Model and data (configs/olmoe_1b7b.yaml): vocab 50304, d_model 2048, 16 layers, 16 heads, seq 4096, 64 SwiGLU
experts (F 1024) per layer, top-8, aux-loss coefficient 0.01, bf16 compute with fp32 master weights, AdamW,
random-init weights N(0, 0.02), synthetic uniform-random token ids.  Weak scaling: every GPU processes 32
sequences (131,072 tokens) per optimizer step as 8 microbatches of 4, so 8 GPUs make the 1M-token global batch;
parallelism is sharded data parallel dp=N with the expert-parallel group ep=N carved from it.

Two timed regions of K steps each, both bracketed by a barrier and a device synchronisation and timed with CUDA
events (maximum over ranks):
  * ``value``: inputs already resident on the device;
  * ``e2e``:   through ``Trainer.train_step`` with the step's token ids copied from pinned host memory every step
               and the step loss read back to the host every step.
Rank 0 prints one JSON line.  ``--impl reference`` runs the unmodified reference package installed under
``baseline/_ref`` (its ToyMoEModel + train-loop recipe) on the same shapes and prints the same line with
``"impl": "reference"``, or an ``unavailable`` line when it cannot run.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

SEQS_PER_GPU = 32
MICRO_BATCH = 4


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference", "library"], default="ours",
                    help="ours: this repository's kernels; reference: the unmodified reference package; library: this "
                         "repository's model with every hot op on NVIDIA / PyTorch library kernels (cuBLAS per expert, "
                         "NCCL all-to-all, fused attention from the library, eager norms, torch.optim.AdamW)")
    ap.add_argument("--config", default=str(ROOT / "configs" / "olmoe_1b7b.yaml"))
    ap.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--keep-mesh", action="store_true",
                    help="keep the configuration's own dp / ep / tp / pp mesh (its world size must equal the number "
                         "of ranks) instead of dp = ep = N; for configurations other than the headline one")
    ap.add_argument("--mesh", default=None, metavar="DP,EP,TP,PP",
                    help="with --keep-mesh: override the configuration's mesh (ep carved from dp), e.g. 1,1,2,2")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (a proxy run, not a headline)")
    ap.add_argument("--ckpt-dir", default=None,
                    help="take one asynchronous checkpoint (pinned snapshot + background write to this directory) "
                         "inside the end-to-end timed region and report what it cost")
    ap.add_argument("--ckpt-step", type=int, default=1, help="index of the timed step after which the checkpoint is taken")
    ap.add_argument("--ckpt-model-only", action="store_true", help="checkpoint the bf16 weights only (no optimizer state)")
    ap.add_argument("--tiny", action="store_true",
                    help="self-test of the reference arm with toy dimensions (runs on CPU too); never a bench value")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of the local GPU with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def max_over_ranks(value: float, device) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        return value
    t = torch.tensor([value], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync():
    import torch
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def timed_region(step_fn, steps: int, device) -> float:
    """Milliseconds for ``steps`` calls of ``step_fn`` measured with CUDA events, maximum over ranks."""
    import torch

    barrier_sync()
    if not torch.cuda.is_available():  # only the toy self-test of the reference arm runs without a GPU
        t0 = time.perf_counter()
        for i in range(steps):
            step_fn(i)
        return max_over_ranks((time.perf_counter() - t0) * 1e3, device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    barrier_sync()
    return max_over_ranks(ms, device)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 1590.0, 1400.0, "fallback"


def run_ours(args) -> dict:
    import torch

    sys.path.insert(0, str(ROOT))
    from composed_mixture_of_experts_engine_b200.engine import Trainer, init_distributed
    from composed_mixture_of_experts_engine_b200.ops import _ext
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig
    from composed_mixture_of_experts_engine_b200.utils.mfu import exact_train_flops_per_token

    library = args.impl == "library"
    if library:
        # every hot op on library kernels: the differentiable ops take their PyTorch paths, the exchanges NCCL
        os.environ["CMOE_FORCE_LIBRARY"] = "1"
        os.environ["CMOE_EP_TRANSPORT"] = os.environ["CMOE_DP_TRANSPORT"] = "nccl"
        os.environ["CMOE_DISABLE_PEER_KERNELS"] = "1"
    rank, world = init_distributed("cuda")
    n = world
    cfg = MoEConfig.from_yaml(args.config)
    d = cfg.to_dict()
    accum = max(1, args.seqs_per_gpu // args.micro_batch)
    if args.layers > 0:
        d["model"]["num_layers"] = args.layers
    if args.keep_mesh and args.mesh:
        dp_, ep_, tp_, pp_ = (int(v) for v in args.mesh.split(","))
        d["parallelism"].update(data_parallel=dp_, expert_parallel=ep_, tensor_parallel=tp_, pipeline_parallel=pp_,
                                ep_from_dp=True)
        cfg = MoEConfig.from_dict(d)
    if args.keep_mesh:
        if cfg.parallelism.world_size != n:
            raise SystemExit(f"--keep-mesh: {args.config} describes {cfg.parallelism.world_size} ranks, started {n}")
        replicas = cfg.parallelism.data_parallel
    else:
        d["parallelism"].update(data_parallel=n, expert_parallel=n, tensor_parallel=1, pipeline_parallel=1,
                                ep_from_dp=True)
        replicas = n
    d["training"].update(micro_batch_size=args.micro_batch, gradient_accumulation_steps=accum,
                         global_batch_size=args.micro_batch * accum * replicas, warmup_steps=0, max_steps=10_000)
    cfg = MoEConfig.from_dict(d)
    trainer = Trainer(cfg)
    dev = trainer.device
    m = cfg.model
    # ranks of one data-parallel replica (tensor / pipeline peers) see the same sequences
    gen = torch.Generator().manual_seed(1234 + (trainer.topology.dp_rank if args.keep_mesh else rank))
    n_batches = 2
    host = [trainer.synthetic_batch(gen, pinned=True) for _ in range(n_batches)]
    resident = [(a.to(dev), b.to(dev)) for a, b in host]

    def dev_step(i):
        ids, tgt = resident[i % n_batches]
        return trainer.train_step(ids, tgt)

    losses = []
    ckpt = None
    if args.ckpt_dir:
        from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import AsyncCheckpointer, LocalNVMeAdapter

        ckpt = AsyncCheckpointer(LocalNVMeAdapter(args.ckpt_dir), None, retention=1, workers=2)
        ckpt.prepare(trainer.model, None if args.ckpt_model_only else trainer.optimizer)  # as train.py does at start-up

    def e2e_step(i):
        ids, tgt = host[i % n_batches]
        loss = trainer.train_step(ids, tgt)  # H2D copy of the pinned batch happens inside
        losses.append(float(loss.item()))     # D2H read of the step result
        if ckpt is not None and i == args.ckpt_step:
            ckpt.save(trainer.model, None if args.ckpt_model_only else trainer.optimizer, 1000 + i, rank=rank,
                      guard_with=trainer.optimizer)

    for i in range(args.warmup):
        dev_step(i)
    torch.cuda.synchronize()
    _ext.reset_launch_counts()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms_dev = timed_region(dev_step, args.steps, dev)
    launches = _ext.launch_counts_total()
    ms_e2e = timed_region(e2e_step, args.steps, dev)
    clocks = sampler.stop()
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status

    check_status(dev)
    # the same step with this package's own attention kernels instead of the library's (or the other way round when
    # CMOE_ATTN_SM100=1 selected them for the main measurement): two untimed steps, then a short timed region
    attn_alt = None
    if not library and not args.keep_mesh:
        main_own = os.environ.get("CMOE_ATTN_SM100", "0") == "1"
        os.environ["CMOE_ATTN_SM100"] = "0" if main_own else "1"
        try:
            for i in range(2):
                dev_step(i)
            k_alt = max(2, min(args.steps, 4))
            ms_alt = timed_region(dev_step, k_alt, dev)
            attn_alt = {"attention": "library (cuDNN fused attention)" if main_own else
                        "hand-written tcgen05 kernels (csrc/attention_fwd2.cu, csrc/attention.cu)",
                        "value": trainer.tokens_per_step_per_rank * n / (ms_alt / k_alt / 1e3), "unit": "tokens/s",
                        "steps": k_alt, "ms_per_step": ms_alt / k_alt}
        finally:
            os.environ["CMOE_ATTN_SM100"] = "1" if main_own else "0"
        check_status(dev)
    ckpt_info = None
    if ckpt is not None:
        t0 = time.perf_counter()
        ckpt.shutdown(drain=True)  # outside the timed region: wait for the background write to finish
        files = list(Path(args.ckpt_dir).rglob(f"rank={rank:06d}.pt"))
        ckpt_info = {"async_ckpt_commit_ms": ckpt.last_commit_ms, "snapshot_d2h_ms": ckpt.last_d2h_ms,
                     "background_write_ms": ckpt.last_write_ms, "drain_wait_after_timing_s": time.perf_counter() - t0,
                     "bytes_this_rank": files[0].stat().st_size if files else 0,
                     "what": "bf16 weights" if args.ckpt_model_only else "bf16 weights + fp32 master / moments shard",
                     "error": repr(ckpt.last_error) if ckpt.last_error else None}

    tokens_step = trainer.tokens_per_step_global if args.keep_mesh else trainer.tokens_per_step_per_rank * n
    per_step_ms = ms_dev / args.steps
    value = tokens_step / (per_step_ms / 1e3)
    e2e_value = tokens_step / (ms_e2e / args.steps / 1e3)
    flops_tok = exact_train_flops_per_token(m.hidden_dim, m.num_layers, m.ffn_dim, m.num_experts, m.top_k,
                                            m.sequence_length, m.vocab_size, m.resolved_num_heads,
                                            m.resolved_num_kv_heads, m.resolved_head_dim)
    burst, sustained, how = peaks()
    achieved_tflops = flops_tok * value / 1e12
    ids0 = host[0][0]
    out = {
        "metric": "moe_train_tokens_per_sec",
        "value": value,
        "unit": "tokens/s",
        "n_gpus": n,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": per_step_ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform-random token ids; random-init weights N(0,0.02)",
        "impl": args.impl,
        "config": {
            "model": ("OLMoE-1B-7B-shaped (V50304 d2048 L16 h16 S4096 E64 F1024 top8, aux 0.01)"
                      if Path(args.config).name == "olmoe_1b7b.yaml" else
                      f"{Path(args.config).stem} (V{m.vocab_size} d{m.hidden_dim} L{m.num_layers} "
                      f"h{m.resolved_num_heads}/{m.resolved_num_kv_heads} S{m.sequence_length} E{m.num_experts} "
                      f"F{m.ffn_dim} top{m.top_k})"),
            "global_batch": args.micro_batch * accum * replicas,
            "global_batch_tokens": tokens_step,
            "seq_len": m.sequence_length,
            "micro_batch": args.micro_batch,
            "grad_accum": accum,
            "parallelism": (f"dp{n} x ep{n} (ep carved from dp), sharded optimizer state" if not args.keep_mesh else
                            f"dp{cfg.parallelism.data_parallel} x ep{cfg.parallelism.expert_parallel} x "
                            f"tp{cfg.parallelism.tensor_parallel} x pp{cfg.parallelism.pipeline_parallel}"),
            "optimizer": ("torch.optim.AdamW on the bf16 parameters, clip_grad_norm_ 1.0" if library else
                          "AdamW fp32 master + moments, global-norm clip 1.0"),
            "attention": ("hand-written tcgen05 kernels (CMOE_ATTN_SM100=1)"
                          if os.environ.get("CMOE_ATTN_SM100", "0") == "1" and not library
                          else "library (cuDNN fused attention)"),
            "dense_gemms": ("library (cuBLAS through F.linear)" if library else
                            "hand-written two-SM tcgen05 GEMM (attention projections, LM head: forward, input and "
                            "weight gradients)"),
            "experts_and_exchange": ("library: cuBLAS per expert, NCCL all-to-all" if library else
                                     "grouped tcgen05 GEMMs with the dispatch / combine transfers inside them"),
            "l2": "no explicit flush: every microbatch streams 13.8 GB of bf16 weights and >1 GB of activations "
                  "per layer, far larger than the 126 MB L2",
        },
        "mfu": {"flops_per_token": flops_tok, "achieved_tflops_per_gpu": achieved_tflops / n,
                "of_burst_peak": achieved_tflops / n / burst, "of_sustained_peak": achieved_tflops / n / sustained,
                "peaks": how},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": int(2 * ids0.numel() * ids0.element_size()), "d2h_bytes_per_step": 4,
                "last_loss": losses[-1] if losses else None},
        "gpu_launches": launches,
        "clocks": clocks,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
    }
    if ckpt_info is not None:
        out["checkpoint_in_timed_region"] = ckpt_info
    if attn_alt is not None:
        out["same_step_other_attention"] = attn_alt
    return out if rank == 0 else {}


REFERENCE_DIMS = dict(hidden_dim=2048, num_layers=16, num_experts=64, top_k=8, capacity_factor=1.25, ffn_dim=1024,
                      vocab_size=50304, sequence_length=4096, dtype="bfloat16")
TINY_DIMS = dict(hidden_dim=64, num_layers=2, num_experts=4, top_k=2, capacity_factor=1.25, ffn_dim=128,
                 vocab_size=512, sequence_length=32, dtype="bfloat16")


def _is_oom(exc: BaseException) -> bool:
    return "out of memory" in str(exc).lower()


def run_reference(args) -> dict:
    """The unmodified reference (baseline/_ref/pkg) through its own public API, the way its train.py drives it:
    build_topology -> build_model -> apply_fsdp2 -> torch AdamW, cross entropy on the logits, clip, step
    (reference: train.py:188-325).  None of this repository's models, kernels or engine is on this path."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "pkg").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install missing)"}
    import torch

    # the reference package is called `pkg`: make sure the one under baseline/_ref wins
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref))
    for name in [m for m in sys.modules if m == "pkg" or m.startswith("pkg.")]:
        del sys.modules[name]
    try:
        import torch.distributed as dist
        from pkg.distributed import apply_fsdp2, build_topology
        from pkg.models.moe import build_model
        from pkg.utils.config import MoEConfig as RefConfig

        if not str(Path(sys.modules["pkg"].__file__).resolve()).startswith(str(ref.resolve())):
            return {"impl": "reference", "unavailable": "the reference package under baseline/_ref did not import"}
        tiny = getattr(args, "tiny", False)
        cuda = torch.cuda.is_available()
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        if world > 1:
            if cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
            dist.init_process_group(backend="nccl" if cuda else "gloo", rank=rank, world_size=world)
        dims = dict(TINY_DIMS if tiny else REFERENCE_DIMS)
        seqs = args.seqs_per_gpu
        V, S = dims["vocab_size"], dims["sequence_length"]

        def make_cfg(micro):
            accum = max(1, seqs // micro)
            return RefConfig.from_dict({
                "model": dims,
                "training": dict(global_batch_size=micro * accum * world, micro_batch_size=micro, learning_rate=4e-4,
                                 weight_decay=0.1, grad_clip=1.0, max_steps=10000, warmup_steps=0,
                                 gradient_accumulation_steps=accum),
                # the reference cannot run expert parallelism > 1 (its first all-to-all raises); data parallel only
                "parallelism": dict(data_parallel=world, expert_parallel=1, tensor_parallel=1, pipeline_parallel=1),
                "checkpoint": dict(local_dir="/tmp/ref-ckpt", remote_uri="file:///tmp/ref-remote"),
            })

        cfg = make_cfg(args.micro_batch)
        topo = build_topology(dp_size=world, ep_size=1, tp_size=1, pp_size=1, device_type="cuda" if cuda else "cpu")
        dev = topo.device
        model = build_model(cfg, topo)
        model = apply_fsdp2(model, topo, mixed_precision_dtype=torch.bfloat16 if dims["dtype"] == "bfloat16" else None)
        optim = torch.optim.AdamW(model.parameters(), lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95))
        gen = torch.Generator().manual_seed(1234 + rank)

        def pinned(t):
            return t.pin_memory() if cuda else t

        host = [(pinned(torch.randint(0, V, (seqs, S), generator=gen)),
                 pinned(torch.randint(0, V, (seqs, S), generator=gen))) for _ in range(2)]
        resident = [(a.to(dev), b.to(dev)) for a, b in host]
        micro = [args.micro_batch]

        def step(ids_all, tgt_all):
            B = micro[0]
            accum = max(1, seqs // B)
            optim.zero_grad(set_to_none=True)
            total = 0.0
            for a in range(accum):
                ids, tgt = ids_all[a * B:(a + 1) * B], tgt_all[a * B:(a + 1) * B]
                logits = model(ids)
                loss = torch.nn.functional.cross_entropy(logits.view(-1, V).float(), tgt.reshape(-1)) / accum
                loss.backward()
                total = total + loss.detach()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            optim.step()
            return total

        def dev_step(i):
            return step(*resident[i % 2])

        losses = []

        def e2e_step(i):
            a, b = host[i % 2]
            loss = step(a.to(dev, non_blocking=True), b.to(dev, non_blocking=True))
            losses.append(float(loss.item()))

        # the reference's experts materialise per-expert activations; halve the micro-batch (same tokens per
        # step, more accumulation) until one step fits
        while True:
            try:
                dev_step(0)
                break
            except Exception as exc:
                if not _is_oom(exc) or micro[0] == 1 or world > 1:
                    raise
                micro[0] //= 2
                optim.zero_grad(set_to_none=True)
                del exc
                torch.cuda.empty_cache()
        for i in range(1, args.warmup):
            dev_step(i)
        sampler = None
        if cuda:
            torch.cuda.synchronize()
            sampler = ClockSampler(torch.cuda.current_device())
            sampler.start()
        ms_dev = timed_region(dev_step, args.steps, dev)
        ms_e2e = timed_region(e2e_step, args.steps, dev)
        clocks = sampler.stop() if sampler is not None else {}
        tokens_step = seqs * S * world
        out = {
            "metric": "moe_train_tokens_per_sec", "value": tokens_step / (ms_dev / args.steps / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dims["dtype"] == "bfloat16" else "fp32",
            "data": "synthetic uniform-random token ids; reference default init",
            "impl": "reference",
            "config": {"model": "reference ToyMoEModel with OLMoE-1B-7B dimensions (it has no attention / RoPE)"
                       if not tiny else "reference ToyMoEModel, tiny dimensions (self-test)",
                       "global_batch": seqs * world, "micro_batch": micro[0], "seq_len": S,
                       "parallelism": f"dp{world} (FSDP2), ep1: the reference cannot run ep>1",
                       "l2": "inputs and weights far larger than L2"},
            "e2e": {"value": tokens_step / (ms_e2e / args.steps / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(2 * host[0][0].numel() * 8), "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "clocks": clocks,
        }
        return out if rank == 0 else {}
    except Exception as exc:  # the reference arm must never take the benchmark down
        msg = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
        return {"impl": "reference", "unavailable": f"reference run failed: {msg}"}


def main():
    args = parse_args()
    import torch

    if not torch.cuda.is_available() and not (args.impl == "reference" and args.tiny):
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    out = run_reference(args) if args.impl == "reference" else run_ours(args)  # "library" shares run_ours
    rank = int(os.environ.get("RANK", "0"))
    if out and (rank == 0 or "unavailable" in out and rank == 0):
        print(json.dumps(out))
        sys.stdout.flush()
    import torch.distributed as dist

    if dist.is_initialized():
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception:
            pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
