"""``moe`` command line: train | benchmark | validate | info.

Mirrors the reference's typer CLI (scripts/cli.py:79-391): ``train`` validates the config and then either calls
``train.main`` in-process (one process) or launches ``torchrun --standalone`` with the requested number of
processes; ``benchmark`` runs the micro-benchmark suite; ``validate`` checks YAML files or directories of them;
``info`` prints versions, devices and the state of the CUDA extension.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path
from typing import List, Optional

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

try:
    import typer
except Exception:  # pragma: no cover - typer is optional
    typer = None


def _validate_one(path: Path) -> Optional[str]:
    from composed_mixture_of_experts_engine_b200.utils.config import ConfigValidationError, MoEConfig

    try:
        MoEConfig.from_yaml(path)
        return None
    except (ConfigValidationError, FileNotFoundError) as exc:
        return str(exc)


def cmd_validate(paths: List[str]) -> int:
    files: List[Path] = []
    for p in paths:
        pp = Path(p)
        files += sorted(pp.glob("*.yaml")) if pp.is_dir() else [pp]
    bad = 0
    for f in files:
        err = _validate_one(f)
        print(f"{'FAIL' if err else ' ok '}  {f}")
        if err:
            print("      " + err.replace("\n", "\n      "))
            bad += 1
    return 1 if bad else 0


def cmd_train(config: str, nproc: int = 1, max_steps: Optional[int] = None, smoke: bool = False,
              extra: Optional[List[str]] = None) -> int:
    err = _validate_one(Path(config))
    if err:
        print(err, file=sys.stderr)
        return 2
    args = ["--config", config] + (["--max-steps", str(max_steps)] if max_steps is not None else []) + \
           (["--smoke"] if smoke else []) + list(extra or [])
    if nproc <= 1:
        import train

        return train.main(args)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           f"--nproc-per-node={nproc}", str(ROOT / "train.py")] + args
    return subprocess.call(cmd)


def cmd_benchmark(cuda: bool = False, json_out: Optional[str] = None) -> int:
    from benchmarks import run_benchmark

    argv = (["--cuda"] if cuda else []) + (["--json", json_out] if json_out else [])
    return run_benchmark.main(argv)


def cmd_plan(config: str, world: Optional[int] = None) -> int:
    """Per-GPU memory plan of a configuration against the 180 GB of a B200."""
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig
    from composed_mixture_of_experts_engine_b200.utils.memory import format_plan, plan_memory

    plan = plan_memory(MoEConfig.from_yaml(config), world)
    print(format_plan(plan))
    return 0 if plan["fits"] else 1


def cmd_info() -> int:
    import torch

    import composed_mixture_of_experts_engine_b200 as pkg
    from composed_mixture_of_experts_engine_b200.models import list_registered_models
    from composed_mixture_of_experts_engine_b200.ops import _ext

    info = {
        "engine_version": pkg.__version__,
        "torch": torch.__version__,
        "cuda_available": torch.cuda.is_available(),
        "devices": [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())],
        "extension_built": _ext._so_path().exists(),
        "extension_sources": [s.name for s in _ext.sources()],
        "models": list_registered_models(),
        "nccl": torch.distributed.is_nccl_available(),
    }
    print(json.dumps(info, indent=1))
    return 0


if typer is not None:
    app = typer.Typer(add_completion=False, help="B200-native MoE engine")

    @app.command()
    def train(config: str = typer.Option(..., "--config", "-c"), nproc: int = typer.Option(1, "--nproc"),
              max_steps: Optional[int] = typer.Option(None, "--max-steps"), smoke: bool = typer.Option(False, "--smoke")):
        """Validate CONFIG, then train: in this process (--nproc 1) or as NPROC ranks under torchrun on this node."""
        raise typer.Exit(cmd_train(config, nproc, max_steps, smoke))

    @app.command()
    def benchmark(cuda: bool = typer.Option(False, "--cuda"), json_out: Optional[str] = typer.Option(None, "--json")):
        """Router / MoE-layer / token-conservation micro-benchmarks (benchmarks/run_benchmark.py)."""
        raise typer.Exit(cmd_benchmark(cuda, json_out))

    @app.command()
    def plan(config: str = typer.Option(..., "--config", "-c"), world: Optional[int] = typer.Option(None, "--world")):
        """Per-GPU memory plan of CONFIG (weights, optimizer state, activations, transport buffers) against 180 GB."""
        raise typer.Exit(cmd_plan(config, world))

    @app.command()
    def validate(paths: List[str] = typer.Argument(...)):
        """Validate YAML configs (files or directories); exit status 1 if any fails."""
        raise typer.Exit(cmd_validate(paths))

    @app.command()
    def info():
        """Versions, devices, registered models and whether the sm_100a extension is built."""
        raise typer.Exit(cmd_info())


def main() -> int:
    if typer is not None:
        app()
        return 0
    argv = sys.argv[1:]
    if not argv:
        print("usage: cli.py train|benchmark|validate|plan|info ...", file=sys.stderr)
        return 2
    if argv[0] == "validate":
        return cmd_validate(argv[1:])
    if argv[0] == "info":
        return cmd_info()
    if argv[0] == "plan":
        return cmd_plan(argv[argv.index("--config") + 1],
                        int(argv[argv.index("--world") + 1]) if "--world" in argv else None)
    if argv[0] == "benchmark":
        return cmd_benchmark("--cuda" in argv)
    if argv[0] == "train":
        cfg = argv[argv.index("--config") + 1]
        return cmd_train(cfg, smoke="--smoke" in argv)
    return 2


if __name__ == "__main__":
    sys.exit(main())
