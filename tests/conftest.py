"""Shared pytest configuration: markers, CPU/GPU gating and process-group hygiene."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    config.addinivalue_line("markers", "cpu: runs on CPU only")
    config.addinivalue_line("markers", "chaos: fault-injection tests (host-side faults only)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    has_cuda = torch.cuda.is_available()
    n_dev = torch.cuda.device_count() if has_cuda else 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not has_cuda:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n_dev < 2:
            item.add_marker(skip_multi)
    # Collection order of the GPU suites: the attention kernels (the largest hand-written kernels) run after every
    # other suite, and the allocation-free entry point, which shares one device array between calls, runs last; a
    # run that stops at the first failure has then already run everything else.
    late = {"test_gpu_attention.py": 1, "test_zz_no_alloc.py": 2}
    items.sort(key=lambda it: late.get(Path(str(it.fspath)).name, 0))  # stable: the rest keeps its order


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture
def free_port() -> int:
    return find_free_port()


@pytest.fixture(autouse=True)
def _destroy_leaked_process_group():
    yield
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
