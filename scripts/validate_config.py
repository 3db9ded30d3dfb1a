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

    def tag(ok: bool) -> str:
        word = "OK" if ok else "FAIL"
        return f"{GREEN if ok else RED}{word}{RESET}" if colour else word

    files = []
    for a in argv:
        p = Path(a)
        if p.is_dir():
            found = sorted(list(p.glob("*.yaml")) + list(p.glob("*.yml")))
            if not found:
                print(f"[WARN] no *.yaml / *.yml files in {p}")
            files += found
        elif p.is_file():
            files.append(p)
        else:
            print(f"[{tag(False)}] {p}: no such file or directory")
            return 1
    if not files:
        print("nothing to validate")
        return 1
    failed = 0
    for f in files:
        try:
            cfg = MoEConfig.from_yaml(f)
            m, par = cfg.model, cfg.parallelism
            print(f"[{tag(True)}] {f}  H={m.hidden_dim} E={m.num_experts} K={m.top_k} world_size={par.world_size} "
                  f"dtype={m.dtype} arch={m.arch}")
        except ConfigValidationError as exc:
            failed += 1
            print(f"[{tag(False)}] {f}")
            for line in str(exc).splitlines():
                print(f"       {line}")
        except Exception as exc:  # unreadable file, YAML syntax error, ...: a failure of that file, not of the run
            failed += 1
            print(f"[{tag(False)}] {f}: {type(exc).__name__}: {exc}")
    ok = len(files) - failed
    print(f"{ok} of {len(files)} config(s) valid" + (f", {failed} failed" if failed else ""))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
