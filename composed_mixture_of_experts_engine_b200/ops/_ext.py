"""Builds and loads the sm_100a CUDA extension of this package.

The extension lives in ``csrc/`` and is built in-tree (``_build/``) with
``-gencode arch=compute_100a,code=sm_100a``.  A stamp file records a hash of the
sources, so a machine that received a built ``.so`` together with the sources
imports it without compiling again.

``ext()`` returns the module or raises; it never falls back silently: on a
machine with a GPU the CUDA path is the only path of the hot ops.
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import threading
from pathlib import Path
from types import ModuleType
from typing import Optional

_PKG_DIR = Path(__file__).resolve().parent.parent
CSRC_DIR = _PKG_DIR / "csrc"
BUILD_DIR = _PKG_DIR / "_build"
EXT_NAME = "cmoe_sm100a"

_SOURCES = [
    "bindings.cpp",
    "bindings_attention.cpp",
    "bindings_ep.cpp",
    "gemm.cu",
    "gemm2.cu",
    "router.cu",
    "ops.cu",
    "attention.cu",
    "attention_fwd2.cu",
    "ep.cu",
    "noalloc.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]

_lock = threading.Lock()
_module: Optional[ModuleType] = None


def sources() -> list[Path]:
    return [CSRC_DIR / s for s in _SOURCES if (CSRC_DIR / s).exists()]


def _source_hash() -> str:
    h = hashlib.sha256()
    files = sorted(list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.cpp")) + list(CSRC_DIR.glob("*.h")))
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return BUILD_DIR / f"{EXT_NAME}.so"


def _import_so(path: Path) -> ModuleType:
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(EXT_NAME, str(path))
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load extension from {path}")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[EXT_NAME] = mod
    return mod


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the extension for sm_100a if the stamp does not match the sources."""
    stamp = BUILD_DIR / ".srchash"
    want = _source_hash()
    so = _so_path()
    if not force and so.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return so
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    with _build_lock():
        if not force and so.exists() and stamp.exists() and stamp.read_text().strip() == want:
            return so  # another process built it while this one waited
        _compile(cpp_extension, verbose)
        if not so.exists():
            raise RuntimeError(f"extension build did not produce {so}")
        stamp.write_text(want)
    return so


class _build_lock:
    """Inter-process lock on the build directory that dies with its holder (``flock``).

    torch's own build lock is a plain file that outlives a killed build and travels with a copy of the tree; whoever
    finds it waits forever.  Builds are serialised by this lock instead, and a file left behind by torch's lock is
    removed while it is held (nobody else can be building then)."""

    def __enter__(self):
        import fcntl

        self._fh = open(BUILD_DIR / ".flock", "w")
        fcntl.flock(self._fh, fcntl.LOCK_EX)
        stale = BUILD_DIR / "lock"
        if stale.exists():
            stale.unlink()
        return self

    def __exit__(self, *exc):
        import fcntl

        fcntl.flock(self._fh, fcntl.LOCK_UN)
        self._fh.close()
        return False


def _compile(cpp_extension, verbose: bool) -> None:
    cpp_extension.load(
        name=EXT_NAME,
        sources=[str(s) for s in sources()],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[str(CSRC_DIR)],
        build_directory=str(BUILD_DIR),
        verbose=verbose,
        is_python_module=False,
    )


IO_LIB = BUILD_DIR / "libcmoe_io.so"


def build_io_lib(force: bool = False) -> Path:
    """Compile the checkpoint file writer (plain C++, no torch) into ``_build/libcmoe_io.so``."""
    import subprocess

    src = CSRC_DIR / "odirect_writer.cpp"
    if not force and IO_LIB.exists() and IO_LIB.stat().st_mtime >= src.stat().st_mtime:
        return IO_LIB
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", str(CSRC_DIR), str(src), "-o", str(IO_LIB)],
                   check=True)
    return IO_LIB


# kernels launched by one call of each entry point (cudaMemsetAsync calls are not counted)
_KERNELS_PER_CALL = {"moe_plan": 3, "moe_plan_scratch_words": 0}
_launch_counts: dict = {}


class _CountingExt:
    """The extension module with a per-entry-point call counter (what ``bench.py`` reports as launches)."""

    def __init__(self, mod: ModuleType):
        self._mod = mod
        self._cache: dict = {}

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)
            if not callable(raw):
                return raw
            per_call = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, __raw=raw, __name=name, __n=per_call, **kwargs):
                _launch_counts[__name] = _launch_counts.get(__name, 0) + __n
                return __raw(*args, **kwargs)

            self._cache[name] = fn
        return fn


_proxy: Optional[_CountingExt] = None


def ext() -> _CountingExt:
    """The loaded extension module (built on first use if needed)."""
    global _module, _proxy
    if _proxy is not None:
        return _proxy
    with _lock:
        if _module is None:
            so = build()
            _module = _import_so(so)
        if _proxy is None:
            _proxy = _CountingExt(_module)
    return _proxy


def reset_launch_counts() -> None:
    _launch_counts.clear()


def launch_counts() -> dict:
    return dict(_launch_counts)


def launch_counts_total() -> int:
    return int(sum(_launch_counts.values()))


def available() -> bool:
    """True when the extension can be imported (it is built for sm_100a only)."""
    try:
        ext()
        return True
    except Exception:
        return False
