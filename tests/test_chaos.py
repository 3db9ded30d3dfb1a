"""Fault-injection tests: all faults are made on the host (process death, storage stall); no GPU is involved.

Scenario A: a worker SIGKILLs itself mid-run, TorchElastic restarts the group, training resumes from the newest
checkpoint that every rank has, bit-exactly.  Scenario B: the storage layer stalls once; the training thread is not
held and every step is still committed.  (Reference: tests/test_chaos.py + tests/_chaos_worker.py.)"""

import json
import os
import signal
import subprocess
import sys
from pathlib import Path

import pytest

from tests.conftest import find_free_port

pytestmark = [pytest.mark.cpu, pytest.mark.chaos]
WORKER = Path(__file__).resolve().parent / "_chaos_worker.py"


class _RunTimedOut(Exception):
    pass


def _kill_tree(proc) -> None:
    """Kill the launcher and every descendant, also ones that left its process group."""
    import psutil

    try:
        kids = psutil.Process(proc.pid).children(recursive=True)
    except psutil.Error:
        kids = []
    try:
        os.killpg(proc.pid, signal.SIGKILL)
    except ProcessLookupError:
        pass
    for k in kids:
        try:
            k.kill()
        except psutil.Error:
            pass


def _run(tmp_path, budget_s: float = 150.0, **env):
    e = dict(os.environ, CHAOS_DIR=str(tmp_path), GLOO_SOCKET_IFNAME="lo", OMP_NUM_THREADS="1",
             **{k: str(v) for k, v in env.items()})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--max-restarts=2",
           "--rdzv-backend=c10d", f"--rdzv-endpoint=127.0.0.1:{find_free_port()}", "--local-addr", "127.0.0.1",
           "--monitor-interval", "0.5", str(WORKER)]
    log = tmp_path / "launcher.log"
    with open(log, "w") as fh:  # a file, not a pipe: a stray descendant can never keep the test waiting for EOF
        proc = subprocess.Popen(cmd, env=e, stdout=fh, stderr=subprocess.STDOUT, start_new_session=True)
        try:
            proc.wait(timeout=budget_s)
        except subprocess.TimeoutExpired:
            _kill_tree(proc)
            try:
                proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                pass
            raise _RunTimedOut(log.read_text()[-2000:])
    return proc.returncode, log.read_text()


def _run_with_one_retry(tmp_path, **env):
    """The elastic restart path depends on the launcher's rendezvous, which now and then stalls on a loaded host;
    one stalled attempt is retried in a fresh directory (the reference reports ~85 % for its own scenario A)."""
    for attempt in range(2):
        work = tmp_path / f"attempt{attempt}"
        work.mkdir()
        try:
            rc, out = _run(work, **env)
            return work, rc, out
        except _RunTimedOut as exc:
            last = str(exc)
    pytest.fail("chaos run timed out twice:\n" + last)


def _events(tmp_path, rank):
    ev = []
    for f in sorted(tmp_path.glob(f"rank{rank}_gen*.jsonl")):
        ev += [json.loads(l) for l in f.read_text().splitlines()]
    return ev


@pytest.mark.timeout(420)
def test_scenario_a_sigkill_and_restart(tmp_path):
    tmp_path, rc, out = _run_with_one_retry(tmp_path, CHAOS_STEPS=8, CHAOS_KILL_RANK=1, CHAOS_KILL_STEP=3)
    assert rc == 0, out[-3000:]
    for rank in (0, 1):
        ev = _events(tmp_path, rank)
        gens = {e["generation"] for e in ev}
        assert len(gens) >= 2, f"rank {rank} was never restarted: {gens}"
        resumes = [e for e in ev if e["event"] == "resume"]
        assert resumes and all(r["sha"] == r["want_sha"] for r in resumes)  # bit-exact restore
        done = [e for e in ev if e["event"] == "done"]
        assert done, f"rank {rank} never finished"
        last_gen = max(gens)
        steps = [e for e in ev if e["event"] == "step" and e["generation"] == last_gen]
        idx = [s["step"] for s in steps]
        assert idx == sorted(idx) and idx[-1] == 7
        assert steps[-1]["cum_tokens"] == 8 * 8  # token conservation across the restart
    d0 = [e for e in _events(tmp_path, 0) if e["event"] == "done"][-1]
    d1 = [e for e in _events(tmp_path, 1) if e["event"] == "done"][-1]
    assert d0["sha"] == d1["sha"]  # replicas agree after recovery


@pytest.mark.timeout(420)
def test_scenario_b_storage_stall_does_not_block_training(tmp_path):
    tmp_path, rc, out = _run_with_one_retry(tmp_path, CHAOS_STEPS=4, CHAOS_STALL_S=2.0)
    assert rc == 0, out[-3000:]
    ev = _events(tmp_path, 0)
    steps = [e for e in ev if e["event"] == "step"]
    assert [s["step"] for s in steps] == [0, 1, 2, 3]
    assert max(s["save_blocked_ms"] for s in steps) < 1000.0  # save() only enqueues; the stall is on the worker
    kept = sorted(p.name for p in (tmp_path / "ckpts" / "ckpts").iterdir())
    assert kept == [f"step={i:06d}" for i in range(4)]
