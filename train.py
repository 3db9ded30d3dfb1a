"""Training entry point.

    python train.py --config configs/smoke.yaml [--max-steps N] [--smoke] [--profile]
                    [--prometheus-port P] [--wandb-project NAME] [--no-wandb]
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 train.py --config configs/olmoe_1b7b.yaml

Same flags, YAML schema, telemetry envelope and checkpoint layout as the reference's train.py
(train.py:70-100, 121-483).  The loop itself lives in ``Trainer.train_step``; this file wires config ->
trainer -> telemetry -> elastic harness (asynchronous checkpoints, resume, health checks).  Unlike the
reference loop, nothing here waits for the GPU except when a record is emitted (every ``log_interval`` steps).
"""

from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import ElasticConfig, ElasticTrainerHarness  # noqa: E402
from composed_mixture_of_experts_engine_b200.engine import Trainer, lr_at  # noqa: E402
from composed_mixture_of_experts_engine_b200.telemetry.logger import StepRecord, StructuredLogger  # noqa: E402
from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig, load_config  # noqa: E402
from composed_mixture_of_experts_engine_b200.utils.mfu import (MFUAccountant, compute_moe_flops,  # noqa: E402
                                                                exact_train_flops_per_token)

log = logging.getLogger("train")


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description="MoE training (B200-native engine)")
    ap.add_argument("--config", type=str, default=str(ROOT / "configs" / "default.yaml"))
    ap.add_argument("--max-steps", type=int, default=None, help="override training.max_steps")
    ap.add_argument("--smoke", action="store_true", help="shrink the model to toy dimensions and run 5 steps")
    ap.add_argument("--profile", action="store_true", help="write per-step timings to benchmarks/run_<ts>_rank0.json")
    ap.add_argument("--prometheus-port", type=int, default=0)
    ap.add_argument("--wandb-project", type=str, default=None)
    ap.add_argument("--no-wandb", action="store_true")
    ap.add_argument("--cpu", action="store_true", help="force the CPU / gloo path even when a GPU is present")
    return ap.parse_args(argv)


def _get_lr(step: int, cfg: MoEConfig) -> float:
    t = cfg.training
    return lr_at(step, t.learning_rate, t.warmup_steps, t.max_steps)


def _smoke_config(cfg: MoEConfig) -> MoEConfig:
    d = cfg.to_dict()
    d["model"].update(hidden_dim=64, num_layers=2, ffn_dim=128, num_experts=4, top_k=min(2, d["model"]["top_k"]),
                      sequence_length=16, vocab_size=256, num_heads=2, num_kv_heads=0, head_dim=0)
    d["training"].update(micro_batch_size=2, gradient_accumulation_steps=1, max_steps=5, warmup_steps=0,
                         log_interval=1, ckpt_interval=2, global_batch_size=2)
    d["parallelism"].update(tensor_parallel=1, pipeline_parallel=1)
    return MoEConfig.from_dict(d)


def _check_kernel_status(trainer: Trainer) -> None:
    """Raise ``KernelTimeoutError`` if any kernel since the last check gave up on a bounded wait (a peer that never
    arrived, a tile that never landed): from that step on the exchanged rows cannot be trusted, so the run must
    not go on training on them, let alone checkpoint them over the last good state."""
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status

    check_status(trainer.device)


def _routing_block(trainer: Trainer, cfg: MoEConfig, mfu: float) -> dict:
    """Telemetry of the first MoE layer of this rank (one device read)."""
    layers = trainer.model.moe_layers() if hasattr(trainer.model, "moe_layers") else []
    out = {"kernel": {}, "collective": {}, "routing": {}, "extra": {}}
    if not layers:
        return out
    layer = layers[0]
    prof = layer.router.last_profile
    E, K = cfg.model.num_experts, cfg.model.top_k
    if prof is not None:
        out["kernel"] = {
            "sram_bytes_per_block": prof.sram_bytes_per_block,
            "achieved_bw_gbps": prof.achieved_bandwidth_gbps,
            "tokens_per_expert_mean": prof.tokens_per_expert_mean,
            "tokens_per_expert_std": prof.tokens_per_expert_std,
            "used_triton": False,
            "used_fused_kernel": prof.used_fused_kernel,
            "backend": prof.backend,
            "kernel_ms": prof.kernel_ms,
        }
        counts = prof.dispatch_counts or []
        active = sum(1 for c in counts if c > 0)
        n_tokens = sum(counts) / max(K, 1)
        cap = max(1.0, cfg.model.capacity_factor * n_tokens * K / max(E, 1))
        out["routing"] = {"expert_load_imbalance": prof.expert_load_imbalance, "router_z_loss": prof.router_z_loss,
                          "aux_loss": prof.aux_loss}
        out["extra"] = dict(sparse_mfu=mfu * K / max(E, 1), dead_expert_count=len(counts) - active,
                            routing_efficiency=(sum(counts) / (cap * E)) if counts else 0.0, active_experts=active,
                            dropped_token_fraction=layer.last_dropped_token_fraction)
    out["collective"] = {
        "all_to_all_dispatch_ms": layer.last_dispatch_ms,
        "all_to_all_combine_ms": layer.last_combine_ms,
        "expert_compute_ms": layer.last_expert_compute_ms,
        "comm_compute_overlap_ratio": layer.last_overlap_ratio,
    }
    return out


def main(argv=None) -> int:
    args = parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    cfg = load_config(args.config).typed()
    if args.smoke:
        cfg = _smoke_config(cfg)
    if args.max_steps is not None:
        d = cfg.to_dict()
        d["training"]["max_steps"] = args.max_steps
        d["training"]["warmup_steps"] = min(d["training"]["warmup_steps"], max(args.max_steps - 1, 0))
        cfg = MoEConfig.from_dict(d)

    trainer = Trainer(cfg, device_type="cpu" if args.cpu else None)
    topo = trainer.topology
    rank = topo.rank
    t, m = cfg.training, cfg.model

    logger = StructuredLogger(
        json_path=cfg.telemetry.json_path if topo.world_size == 1 else
        str(Path(cfg.telemetry.json_path).with_suffix(f".rank{rank}.jsonl")),
        tensorboard_dir=cfg.telemetry.tensorboard_dir, rank=rank, also_stdout=True,
        prometheus_port=args.prometheus_port, wandb_enabled=not args.no_wandb,
        wandb_init_kwargs={"project": args.wandb_project} if args.wandb_project else None)
    logger.log_config(cfg.to_dict())

    if rank == 0:
        from composed_mixture_of_experts_engine_b200.utils.memory import format_plan, plan_memory

        plan = plan_memory(cfg, topo.world_size, mesh=(topo.dp_size, topo.ep_size, topo.tp_size, topo.pp_size,
                                                       topo.ep_from_dp))
        on_gpu = topo.device.type == "cuda"
        (log.warning if on_gpu and not plan["fits"] else log.info)("memory plan per GPU\n%s", format_plan(plan))

    is_decoder = m.arch == "moe_decoder"
    if is_decoder:
        flops_per_token = exact_train_flops_per_token(m.hidden_dim, m.num_layers, m.ffn_dim, m.num_experts, m.top_k,
                                                      m.sequence_length, m.vocab_size, m.resolved_num_heads,
                                                      m.resolved_num_kv_heads, m.resolved_head_dim)
    else:
        flops_per_token = compute_moe_flops(m.hidden_dim, m.num_layers, m.ffn_dim, m.num_experts, m.top_k,
                                            m.sequence_length, batch_tokens=1, vocab_size=m.vocab_size)
    mfu_acct = MFUAccountant(peak_tflops=cfg.telemetry.hardware_peak_tflops, mfu_target=cfg.telemetry.mfu_target)
    mfu_acct.configure(flops_per_token)

    harness = ElasticTrainerHarness(
        ElasticConfig(local_ckpt_dir=cfg.checkpoint.local_dir, remote_uri=cfg.checkpoint.remote_uri,
                      s3_endpoint=os.environ.get("S3_ENDPOINT_URL"), retention=cfg.checkpoint.retention,
                      async_workers=cfg.checkpoint.async_workers,
                      health_interval_s=cfg.elastic.health_check_interval_s,
                      drop_grace_s=cfg.elastic.drop_grace_period_s, min_nodes=cfg.elastic.min_nodes), topo)
    harness.install_signal_handlers()
    if trainer.device.type == "cuda" and t.ckpt_interval > 0:
        # pin the host staging buffers of the asynchronous checkpoints now, not inside the first save
        pinned = harness.async_ckpt.prepare(trainer.model, trainer.optimizer)
        log.info("pinned %.1f GB of host memory for checkpoint snapshots", pinned / 1e9)

    start_step = 0
    try:
        latest = harness.resume(trainer.model, trainer.optimizer, m.num_experts)
        if latest is not None:
            start_step = latest + 1
            log.info("resumed from step %d", latest)
    except Exception as exc:
        log.warning("could not resume (%s); starting fresh", exc)
    trainer.step_index = start_step

    # one data stream per data replica: tensor- and pipeline-parallel peers of a replica must see the same tokens
    gen = torch.Generator().manual_seed(t.seed + 7919 * topo.data_rank + 104729 * start_step)
    for layer in (trainer.model.moe_layers() if hasattr(trainer.model, "moe_layers") else [])[:1]:
        layer.enable_timing(True)
        layer.router.profile_timing = True
    profile_rows = []
    tokens_per_step = trainer.tokens_per_step_per_rank
    use_cuda = trainer.device.type == "cuda"
    t_log = time.perf_counter()
    steps_since_log = 0
    loss_t: Optional[torch.Tensor] = None

    for step in range(start_step, t.max_steps):
        mfu_acct.start_step()
        ids, tgt = trainer.synthetic_batch(gen)
        loss_t = trainer.train_step(ids, tgt)
        steps_since_log += 1
        do_log = (step % max(t.log_interval, 1) == 0) or step == t.max_steps - 1
        if do_log:
            loss = float(loss_t)  # the only host wait of the loop
            if use_cuda:
                torch.cuda.synchronize()
                _check_kernel_status(trainer)  # a bounded device wait that ran out must stop the run here
            now = time.perf_counter()
            dt = (now - t_log) / steps_since_log
            t_log, steps_since_log = now, 0
            res = mfu_acct.end_step(tokens_per_step, step_time_sec=dt)
            blocks = _routing_block(trainer, cfg, res.mfu)
            rec = StepRecord(
                step=step, loss=loss, mfu=res.mfu, tokens_per_sec=res.tokens_per_sec * topo.data_replicas,
                kernel=blocks["kernel"], collective=blocks["collective"],
                infra={"async_ckpt_commit_ms": harness.async_ckpt.last_commit_ms,
                       "async_ckpt_d2h_ms": harness.async_ckpt.last_d2h_ms,
                       "async_ckpt_write_ms": harness.async_ckpt.last_write_ms,
                       "active_nodes": len(harness.state.alive_ranks()), "ep_world_size": topo.ep_size,
                       "lr": _get_lr(step, cfg), "grad_accum": t.gradient_accumulation_steps},
                routing=blocks["routing"], wall_clock_ms=dt * 1e3, **blocks["extra"])
            logger.emit(rec)
            if args.profile:
                profile_rows.append({"step": step, "step_ms": dt * 1e3, "tokens_per_sec": rec.tokens_per_sec,
                                     "mfu": res.mfu, "loss": loss, **blocks["collective"]})
        if t.ckpt_interval > 0 and step > 0 and step % t.ckpt_interval == 0:
            if use_cuda:
                _check_kernel_status(trainer)  # never write weights that a timed-out exchange may have corrupted
            harness.checkpoint(trainer.model, trainer.optimizer, step)
        if step > 0 and step % 50 == 0:
            dead = harness.health_check()
            if dead:
                log.warning("ranks %s stopped answering; recovering", dead)

                def _rebuild(new_topology):
                    # another expert-parallel degree means other expert tensors per rank: build the trainer anew
                    nonlocal trainer
                    trainer = Trainer(cfg, topology=new_topology)
                    return trainer.model, trainer.optimizer

                new_topo = harness.recover(trainer.model, trainer.optimizer, m.num_experts, rebuild=_rebuild)
                trainer.topology = new_topo

    if t.max_steps > start_step:
        if use_cuda:
            _check_kernel_status(trainer)
        harness.checkpoint(trainer.model, trainer.optimizer, t.max_steps)
    harness.shutdown()
    logger.close()
    if args.profile and rank == 0 and profile_rows:
        out_dir = Path(os.environ.get("MOE_PROFILE_DIR", str(ROOT / "benchmarks")))
        out_dir.mkdir(parents=True, exist_ok=True)
        ms = sorted(r["step_ms"] for r in profile_rows)
        summary = {"steps": profile_rows, "mean_step_ms": sum(ms) / len(ms), "p50_step_ms": ms[len(ms) // 2],
                   "mfu_summary": mfu_acct.summary_str()}
        (out_dir / f"run_{int(time.time())}_rank0.json").write_text(json.dumps(summary, indent=1))
    log.info("done: %s", mfu_acct.summary_str())
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
