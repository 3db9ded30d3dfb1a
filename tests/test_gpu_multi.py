"""Multi-GPU paths (one process per GPU, NCCL): expert parallelism on the device path and the sharded optimizer.

Runs only where at least two CUDA devices are visible.  Oracles are single-GPU computations of the same math."""

import math

import pytest
import torch
import torch.multiprocessing as mp

from tests import _mp_workers
from tests.conftest import find_free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _spawn_gpu(fn_name, world, *args, timeout=600):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = find_free_port()
    procs = [ctx.Process(target=_mp_workers.run, args=(fn_name, r, world, port, q, args, "nccl")) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        import queue as _queue
        import time as _time

        deadline = _time.time() + timeout
        while len(results) < world:
            try:
                rank, status, payload = q.get(timeout=2.0)
            except _queue.Empty:
                dead = [p.pid for p in procs if p.exitcode not in (None, 0)]
                assert not dead, f"worker process(es) {dead} died without reporting (exit codes " \
                                 f"{[p.exitcode for p in procs]})"
                assert _time.time() < deadline, "timed out waiting for the workers"
                continue
            assert status == "ok", f"rank {rank} failed:\n{payload}"
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return results


def _world():
    n = torch.cuda.device_count()
    return 4 if n >= 4 else 2


@pytest.mark.parametrize("transport", ["nccl", "auto", "auto-pull", "auto-debug"])
def test_ep_layer_matches_single_gpu(transport):
    res = _spawn_gpu("gpu_ep_layer", _world(), transport)
    for r, out in res.items():
        assert out.pop("replay") == 0.0, (r, "the same inputs twice gave different bits")
        for k, v in out.items():
            tol = 6e-2 if k.startswith("dgate") else 3e-2
            assert v < tol, (r, k, v, out)


@pytest.mark.parametrize("transport", ["nccl", "auto"])
def test_trainer_multi_gpu(transport):
    res = _spawn_gpu("gpu_trainer", _world(), transport, 8)
    for r, out in res.items():
        assert all(math.isfinite(l) for l in out["losses"]) and out["losses"][-1] < out["losses"][0]
        assert out["sync"] == 0.0 and out["ep"] == _world()


@pytest.mark.parametrize("transport", ["auto", "auto-pull"])
def test_sequence_parallel_linears_on_peer_memory(transport):
    res = _spawn_gpu("gpu_tp_sp", 2, transport)
    for r, out in res.items():
        for k, v in out.items():
            assert v < 4e-2, (r, k, v, out)


def test_moe_layer_takes_sequence_shards_over_the_ep_x_tp_block():
    """tp = 2 (and ep = 2 with four GPUs): every (expert, FFN slice) pair is an expert of its own in the exchange, so the
    sequence gather and the reduce-scatter around the layer happen inside its grouped GEMM kernels."""
    world = _world()
    ep = world // 2
    res = _spawn_gpu("gpu_moe_sequence_shard", world, ep, 2)
    for r, out in res.items():
        assert out.pop("fused")
        for k, v in out.items():
            tol = 6e-2 if k.startswith("dgate") else 3e-2
            assert v < tol, (r, k, v, out)


def test_trainer_tensor_sequence_parallel_on_gpus():
    """tp = 2 with sequence parallelism (no pipeline): the MoE blocks take sequence shards over peer memory, the
    attention projections gather / reduce-scatter inside their GEMMs.  The loss falls, and every parameter that both
    ranks hold whole (norms, router gate, embedding, LM head) is bit-identical on both after training, which it can
    only be if the partial gradients of the two sequence shards were summed before each update."""
    res = _spawn_gpu("gpu_trainer_hybrid", 2, 1, 1, 2, 1, 8)
    a, b = res[0], res[1]
    assert a["fused_sp_moe"] and b["fused_sp_moe"]
    assert all(math.isfinite(l) for l in a["losses"]) and a["losses"][-1] < a["losses"][0]
    assert a["losses"] == b["losses"]
    for name in a["whole"]:
        assert a["whole"][name] == b["whole"][name], name


def test_trainer_pipeline_parallel_on_gpus():
    """Two pipeline stages over NCCL (1F1B, 4 microbatches), bf16 kernels and the fused optimizer on every stage; with
    four GPUs also tensor + sequence parallelism inside each stage."""
    world = _world()
    tp = 2 if world == 4 else 1
    res = _spawn_gpu("gpu_trainer_hybrid", world, 1, 1, tp, 2, 8)
    last = [out for out in res.values() if out["last"]]
    assert len(last) == world // 2 and all(out["n_blocks"] == 2 for out in res.values())
    for out in last:
        assert all(math.isfinite(l) for l in out["losses"]) and out["losses"][-1] < out["losses"][0]
