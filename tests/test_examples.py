"""Every script under examples/ runs to completion on CPU (the reference ships the first seven as its user-facing
walkthroughs, examples/01..07 there; its tests do not run them)."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
EXAMPLES = sorted((ROOT / "examples").glob("0*.py"))


@pytest.mark.parametrize("script", EXAMPLES, ids=[p.stem for p in EXAMPLES])
def test_example_runs(script, tmp_path):
    out = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300, cwd=str(ROOT),
                         env={**os.environ, "CUDA_VISIBLE_DEVICES": "", "TMPDIR": str(tmp_path)})
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-1500:]
