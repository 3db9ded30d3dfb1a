"""Structured telemetry: one StepRecord fanned out to JSONL (+ stdout / TensorBoard / Prometheus / WandB)."""
import json
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from composed_mixture_of_experts_engine_b200.telemetry import PhaseTimer, StepRecord, StructuredLogger

with tempfile.TemporaryDirectory() as d:
    logger = StructuredLogger(json_path=f"{d}/step.jsonl", tensorboard_dir=None, rank=0, also_stdout=False,
                              wandb_enabled=False)
    timer = PhaseTimer()
    for step in range(3):
        with timer.phase("dispatch"):
            sum(range(10000))
        times = timer.resolve()
        logger.emit(StepRecord(step=step, loss=5.0 - step, mfu=0.41, tokens_per_sec=7.5e4,
                               collective={"all_to_all_dispatch_ms": times.get("dispatch", 0.0)},
                               routing={"expert_load_imbalance": 1.1}, sparse_mfu=0.41 * 8 / 64, active_experts=64))
    logger.close()
    lines = Path(f"{d}/step.jsonl").read_text().splitlines()
    rec = json.loads(lines[-1])
    print("records:", len(lines), "| keys:", sorted(rec))
    print("routing block:", rec["routing"])
