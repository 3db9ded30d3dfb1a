"""Validate one or more YAML configs (files or directories) and print a coloured verdict per file.

    python scripts/validate_config.py configs/ other.yaml

Exit status 1 when any file fails (reference: scripts/validate_config.py)."""

from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

GREEN, RED, RESET = "\033[32m", "\033[31m", "\033[0m"


def main(argv=None) -> int:
    from composed_mixture_of_experts_engine_b200.utils.config import ConfigValidationError, MoEConfig

    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print("usage: validate_config.py <file-or-dir> ...", file=sys.stderr)
        return 2
    colour = sys.stdout.isatty()
    files = []
    for a in argv:
        p = Path(a)
        files += sorted(p.glob("*.yaml")) if p.is_dir() else [p]
    failed = 0
    for f in files:
        try:
            cfg = MoEConfig.from_yaml(f)
            tag = f"{GREEN}OK{RESET}" if colour else "OK"
            print(f"[{tag}] {f}  (world_size={cfg.parallelism.world_size}, arch={cfg.model.arch})")
        except (ConfigValidationError, FileNotFoundError) as exc:
            failed += 1
            tag = f"{RED}FAIL{RESET}" if colour else "FAIL"
            print(f"[{tag}] {f}\n{exc}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
