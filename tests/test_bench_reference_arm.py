"""The benchmark's reference arm: the unmodified reference package under baseline/_ref, driven through its own
public API.  Runs the toy-dimension self-test on CPU; skipped when the reference is not installed."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "pkg").exists(), reason="reference not installed")
def test_reference_arm_prints_one_json_line_with_the_reference_loaded():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--tiny", "--steps", "2",
                          "--warmup", "1", "--seqs-per-gpu", "4", "--micro-batch", "2"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and "unavailable" not in rec, rec
    assert rec["value"] > 0 and rec["e2e"]["value"] > 0 and rec["e2e"]["h2d_bytes_per_step"] == 2 * 4 * 32 * 8


def test_reference_arm_without_a_gpu_reports_unavailable_and_exits_zero():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup",
                          "1"], capture_output=True, text=True, timeout=600, cwd=str(ROOT),
                         env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == 0
    rec = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert rec["impl"] == "reference" and "unavailable" in rec


def test_loss_curves_fall_together_with_the_reference():
    """Equal weights, equal batches, equal optimizer: both curves fall and stay close (the reference's layer picks
    experts by row position, so the curves are near, not identical)."""
    if not (ROOT / "baseline" / "_ref" / "pkg").is_dir():
        pytest.skip("baseline/_ref is not installed")
    out = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "loss_parity.py"), "--steps", "60"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    ref_first, ours_first = line["first_loss"]
    ref_last, ours_last = line["last_loss"]
    assert abs(ref_first - ours_first) < 0.1
    assert ref_last < ref_first - 0.5 and ours_last < ours_first - 0.5
    assert line["max_abs_diff"] < 0.5

