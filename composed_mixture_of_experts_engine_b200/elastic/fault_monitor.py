"""Two-tier asynchronous checkpointing, rank-liveness state machine and the elastic training harness.

Public surface of the reference's ``pkg/elastic/fault_monitor.py`` (``ObjectStoreAdapter``,
``LocalNVMeAdapter``, ``S3Adapter``, ``AsyncCheckpointer``, ``ClusterStateMachine``, ``ElasticConfig``,
``ElasticTrainerHarness``, ``_largest_divisor_le``, ``_check_schema_compatibility``,
``CHECKPOINT_SCHEMA_VERSION``) and its on-disk layout, byte for byte:

    <local_dir>/ckpts/step=%06d/rank=%06d.pt          torch.save({"model": ..., "optim": ...})
    <local_dir>/ckpts/step=%06d/rank=%06d.meta.json   schema_version, step, rank, hostname, ts, versions, extras

What is different underneath:

* ``save`` really is non-blocking.  The reference builds the CPU state dict and pickles it on the training
  thread (fault_monitor.py:321-337).  Here CUDA tensors are copied into pinned host buffers on a side stream
  (the training thread only enqueues the copies), and a worker thread waits for the copy event, serialises,
  and writes.  ``last_commit_ms`` keeps its meaning: how long the training thread was held.
* ``LocalNVMeAdapter`` writes through a page-aligned O_DIRECT writer in C++ (``csrc/odirect_writer.cpp``),
  with an atomic tmp -> rename, instead of attempting O_DIRECT on an unaligned ``bytes`` object (:155-189).
* ``ElasticTrainerHarness.recover`` applies the expert re-ownership plan when the expert-parallel degree
  changed: each surviving rank loads the rows of the stacked expert weights it now owns from whichever old
  rank files hold them (the reference computed the plan and threw it away, :833-835).
* Heartbeats never wait on a device: they use the host-side store / a gloo barrier with a timeout.
"""

from __future__ import annotations

import ctypes
import io
import json
import logging
import os
import queue
import signal
import socket
import threading
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from .. import __version__ as _engine_version
from ..parallel.mesh import ParallelTopology, build_topology

log = logging.getLogger(__name__)

try:
    import boto3  # type: ignore
    from botocore.config import Config as BotoConfig  # type: ignore

    _HAS_BOTO3 = True
except Exception:
    boto3 = None  # type: ignore
    BotoConfig = None  # type: ignore
    _HAS_BOTO3 = False

CHECKPOINT_SCHEMA_VERSION = 2

__all__ = [
    "AsyncCheckpointer", "ClusterStateMachine", "ElasticTrainerHarness", "ElasticConfig", "ObjectStoreAdapter",
    "LocalNVMeAdapter", "S3Adapter", "CHECKPOINT_SCHEMA_VERSION", "_largest_divisor_le",
    "_check_schema_compatibility",
]


def _check_schema_compatibility(meta: Dict[str, Any]) -> None:
    """Log (never raise) when a checkpoint was written under another schema version."""
    loaded = int(meta.get("schema_version", 1))
    if loaded > CHECKPOINT_SCHEMA_VERSION:
        log.warning("Checkpoint schema_version=%d is newer than this build (%d); unknown fields are ignored.",
                    loaded, CHECKPOINT_SCHEMA_VERSION)
    elif loaded < CHECKPOINT_SCHEMA_VERSION:
        log.info("Checkpoint schema_version=%d is older than current=%d; missing fields use defaults.",
                 loaded, CHECKPOINT_SCHEMA_VERSION)


# ==================================================================================================
# object stores
# ==================================================================================================
class ObjectStoreAdapter(ABC):
    @abstractmethod
    def put(self, key: str, payload: bytes) -> None: ...

    @abstractmethod
    def get(self, key: str) -> bytes: ...

    @abstractmethod
    def list(self, prefix: str) -> List[str]: ...

    @abstractmethod
    def delete(self, key: str) -> None: ...


_io_lib = None
_io_lib_failed = False


def _load_io_lib():
    global _io_lib, _io_lib_failed
    if _io_lib is not None or _io_lib_failed:
        return _io_lib
    try:
        from ..ops import _ext

        lib = ctypes.CDLL(str(_ext.build_io_lib()))
        lib.cmoe_write_file.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                        ctypes.c_size_t, ctypes.POINTER(ctypes.c_int)]
        lib.cmoe_write_file.restype = ctypes.c_int
        _io_lib = lib
    except Exception as exc:  # pragma: no cover - toolchain dependent
        log.warning("native checkpoint writer unavailable (%s); using buffered Python writes", exc)
        _io_lib_failed = True
    return _io_lib


class LocalNVMeAdapter(ObjectStoreAdapter):
    """Tier 1: a local directory (NVMe).  Writes are tmp-file + fsync + atomic rename."""

    def __init__(self, root: str, use_odirect: bool = True, chunk_bytes: int = 8 << 20):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.use_odirect = use_odirect
        self.chunk_bytes = chunk_bytes
        self.last_write_used_odirect = False

    def _p(self, key: str) -> Path:
        return self.root / key

    def put(self, key: str, payload: bytes) -> None:
        p = self._p(key)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(p.suffix + ".tmp")
        self._write_chunked(tmp, payload)
        tmp.replace(p)

    def _write_chunked(self, path: Path, payload: bytes, chunk_bytes: Optional[int] = None) -> None:
        lib = _load_io_lib()
        view = memoryview(payload)
        if lib is not None and len(view) > 0:
            used = ctypes.c_int(0)
            if isinstance(payload, bytes):
                buf = payload  # passed by pointer, no copy
            elif view.readonly:
                buf = bytes(view)
            else:
                buf = (ctypes.c_char * len(view)).from_buffer(view)
            rc = lib.cmoe_write_file(str(path).encode(), buf, len(view), 1 if self.use_odirect else 0,
                                     chunk_bytes or self.chunk_bytes, ctypes.byref(used))
            if rc != 0:
                raise OSError(rc, os.strerror(rc), str(path))
            self.last_write_used_odirect = bool(used.value)
            return
        with open(path, "wb") as fh:
            step = chunk_bytes or self.chunk_bytes
            for off in range(0, len(view), step):
                fh.write(view[off:off + step])
            fh.flush()
            os.fsync(fh.fileno())

    def get(self, key: str) -> bytes:
        return self._p(key).read_bytes()

    def list(self, prefix: str) -> List[str]:
        base = self._p(prefix)
        if base.is_file():
            return [prefix]
        if not base.exists():
            return []
        return sorted(str(p.relative_to(self.root)) for p in base.rglob("*")
                      if p.is_file() and not p.name.endswith(".tmp"))

    def delete(self, key: str) -> None:
        try:
            self._p(key).unlink()
        except FileNotFoundError:
            pass
        # drop step directories that became empty
        parent = self._p(key).parent
        try:
            if parent != self.root and not any(parent.iterdir()):
                parent.rmdir()
        except OSError:
            pass


class S3Adapter(ObjectStoreAdapter):
    """Tier 2: S3 / MinIO.  Credentials and endpoint come from the environment (``S3_ENDPOINT_URL``)."""

    def __init__(self, uri: str, endpoint_url: Optional[str] = None):
        if not _HAS_BOTO3:
            raise RuntimeError("boto3 is required for S3Adapter")
        if not uri.startswith("s3://"):
            raise ValueError(f"Expected s3:// uri, got {uri}")
        bucket, _, prefix = uri[len("s3://"):].partition("/")
        self.bucket, self.prefix = bucket, prefix.rstrip("/")
        self._client = boto3.client(
            "s3", endpoint_url=endpoint_url or os.environ.get("S3_ENDPOINT_URL"),
            config=BotoConfig(retries={"max_attempts": 8, "mode": "adaptive"}, connect_timeout=10, read_timeout=60,
                              tcp_keepalive=True))

    def _k(self, key: str) -> str:
        return f"{self.prefix}/{key}" if self.prefix else key

    def put(self, key: str, payload: bytes) -> None:
        self._client.put_object(Bucket=self.bucket, Key=self._k(key), Body=bytes(payload))

    def get(self, key: str) -> bytes:
        return self._client.get_object(Bucket=self.bucket, Key=self._k(key))["Body"].read()

    def list(self, prefix: str) -> List[str]:
        keys: List[str] = []
        for page in self._client.get_paginator("list_objects_v2").paginate(Bucket=self.bucket, Prefix=self._k(prefix)):
            for obj in page.get("Contents", []):
                k = obj["Key"]
                keys.append(k[len(self.prefix) + 1:] if self.prefix else k)
        return keys

    def delete(self, key: str) -> None:
        self._client.delete_object(Bucket=self.bucket, Key=self._k(key))


# ==================================================================================================
# asynchronous checkpointer
# ==================================================================================================
@dataclass
class _CheckpointJob:
    step: int
    payload: Any  # bytes, or a (snapshot, event) pair that the worker serialises
    meta: Dict[str, Any]


def _step_of_key(key: str) -> Optional[int]:
    for seg in key.split("/"):
        if seg.startswith("step="):
            try:
                return int(seg.split("=", 1)[1])
            except ValueError:
                return None
    return None


def _torch_dumps(obj: Any) -> bytes:
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


def _torch_loads(payload: bytes) -> Any:
    return torch.load(io.BytesIO(payload), map_location="cpu", weights_only=False)


class _PinnedStager:
    """Copies a nest of tensors to host memory; CUDA tensors go through pinned buffers on a side stream."""

    def __init__(self) -> None:
        self._streams: Dict[int, Any] = {}

    def snapshot(self, obj: Any):
        """Returns (host copy of ``obj``, CUDA event or None).  Only enqueues work; does not wait for the GPU."""
        devices = set()

        def walk(o):
            if isinstance(o, torch.Tensor):
                if o.is_cuda:
                    devices.add(o.device.index)
                    host = torch.empty(o.shape, dtype=o.dtype, device="cpu", pin_memory=True)
                    host.copy_(o.detach(), non_blocking=True)
                    return host
                return o.detach().clone()
            if isinstance(o, dict):
                return {k: walk(v) for k, v in o.items()}
            if isinstance(o, (list, tuple)):
                return type(o)(walk(v) for v in o)
            return o

        if not torch.cuda.is_available():
            return walk(obj), None
        dev = torch.cuda.current_device()
        side = self._streams.setdefault(dev, torch.cuda.Stream(device=dev))
        main = torch.cuda.current_stream(dev)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            host = walk(obj)
            ev = torch.cuda.Event()
            ev.record(side)
        if not devices:
            return host, None
        # later work of the training stream (the next optimizer step) must not overwrite what is being copied
        main.wait_event(ev)
        return host, ev


class AsyncCheckpointer:
    """Background checkpoint streamer: enqueue on the training thread, serialise + write + mirror + prune on workers."""

    def __init__(self, local_adapter: ObjectStoreAdapter, remote_adapter: Optional[ObjectStoreAdapter],
                 retention: int = 8, workers: int = 4):
        self.local, self.remote = local_adapter, remote_adapter
        self.retention = retention
        self._q: "queue.Queue[_CheckpointJob]" = queue.Queue(maxsize=max(1, workers) * 2)
        self._stop = threading.Event()
        self._threads: List[threading.Thread] = []
        self._completed_steps: List[int] = []
        self._lock = threading.Lock()
        self._stager = _PinnedStager()
        self.last_commit_ms = 0.0
        self.last_error: Optional[BaseException] = None
        for i in range(max(1, workers)):
            t = threading.Thread(target=self._worker, name=f"ckpt-writer-{i}", daemon=True)
            t.start()
            self._threads.append(t)

    # ---- state dict helpers ----------------------------------------------------------------------
    @staticmethod
    def _state(model: torch.nn.Module, optimizer) -> Dict[str, Any]:
        return {"model": dict(model.state_dict()), "optim": optimizer.state_dict() if optimizer is not None else {}}

    def save(self, model: torch.nn.Module, optimizer, step: int, rank: int = 0,
             extra_meta: Optional[Dict[str, Any]] = None) -> None:
        t0 = time.perf_counter()
        snapshot, event = self._stager.snapshot(self._state(model, optimizer))
        meta = {
            "schema_version": CHECKPOINT_SCHEMA_VERSION,
            "step": step,
            "rank": rank,
            "hostname": socket.gethostname(),
            "ts": time.time(),
            "moe_engine_version": _engine_version,
            "torch_version": torch.__version__,
        }
        if extra_meta:
            meta.update(extra_meta)
        self._q.put(_CheckpointJob(step=step, payload=(snapshot, event), meta=meta))
        self.last_commit_ms = (time.perf_counter() - t0) * 1000.0

    def latest_step(self) -> Optional[int]:
        steps = [s for s in (_step_of_key(k) for k in self.local.list("ckpts/")) if s is not None]
        return max(steps) if steps else None

    def _fetch(self, key: str) -> bytes:
        try:
            return self.local.get(key)
        except FileNotFoundError:
            if self.remote is None:
                raise
            payload = self.remote.get(key)
            self.local.put(key, payload)  # re-hydrate the fast tier
            return payload

    def load_raw(self, step: int, rank: int = 0) -> Dict[str, Any]:
        return _torch_loads(self._fetch(f"ckpts/step={step:06d}/rank={rank:06d}.pt"))

    def load(self, model: torch.nn.Module, optimizer, step: int, rank: int = 0) -> Dict[str, Any]:
        obj = self.load_raw(step, rank)
        model.load_state_dict(obj["model"], strict=False)
        if optimizer is not None and obj.get("optim"):
            optimizer.load_state_dict(obj["optim"])
        try:
            meta = json.loads(self._fetch(f"ckpts/step={step:06d}/rank={rank:06d}.meta.json").decode("utf-8"))
        except FileNotFoundError:
            meta = {"step": step, "rank": rank, "schema_version": 1}
        _check_schema_compatibility(meta)
        return meta

    def shutdown(self, drain: bool = True) -> None:
        if self._stop.is_set():
            return
        if drain:
            self._q.join()
        self._stop.set()
        for _ in self._threads:
            try:
                self._q.put_nowait(_CheckpointJob(step=-1, payload=b"", meta={}))
            except queue.Full:
                pass
        for t in self._threads:
            t.join(timeout=5.0)

    # ---- worker ----------------------------------------------------------------------------------
    def _worker(self) -> None:
        while not self._stop.is_set():
            try:
                job = self._q.get(timeout=0.5)
            except queue.Empty:
                continue
            if job.step < 0:
                self._q.task_done()
                break
            try:
                payload = job.payload
                if isinstance(payload, tuple):
                    snapshot, event = payload
                    if event is not None:
                        event.synchronize()
                    payload = _torch_dumps(snapshot)
                root = f"ckpts/step={job.step:06d}/rank={job.meta.get('rank', 0):06d}"
                meta_bytes = json.dumps(job.meta).encode("utf-8")
                self.local.put(f"{root}.pt", payload)
                self.local.put(f"{root}.meta.json", meta_bytes)
                if self.remote is not None:
                    self.remote.put(f"{root}.pt", payload)
                    self.remote.put(f"{root}.meta.json", meta_bytes)
                with self._lock:
                    self._completed_steps = sorted(set(self._completed_steps + [job.step]))[-self.retention:]
                self._prune()
            except Exception as exc:  # keep the worker alive; the failure is visible in last_error and the log
                self.last_error = exc
                log.exception("checkpoint commit failed: %s", exc)
            finally:
                self._q.task_done()

    def _prune(self) -> None:
        with self._lock:
            keep = set(self._completed_steps)
        for store in (self.local, self.remote):
            if store is None:
                continue
            for k in store.list("ckpts/"):
                s = _step_of_key(k)
                if s is not None and s not in keep:
                    try:
                        store.delete(k)
                    except Exception:
                        continue


# ==================================================================================================
# cluster state machine
# ==================================================================================================
@dataclass
class _RankHealth:
    rank: int
    last_heartbeat: float
    alive: bool = True


class ClusterStateMachine:
    """Tracks rank liveness and the phases of an elastic recovery (running -> draining -> recovering -> resumed).

    Liveness is probed on the host only: a store-based heartbeat when a ``store`` is given (every rank bumps its
    own key; a key that stops moving for longer than the grace period marks its rank dead), else a
    ``monitored_barrier`` / barrier with the grace period as its timeout on a gloo group.  No probe ever
    launches a device kernel that waits.
    """

    PHASE_RUNNING = "running"
    PHASE_DRAINING = "draining"
    PHASE_RECOVERING = "recovering"
    PHASE_RESUMED = "resumed"

    def __init__(self, topology: ParallelTopology, health_interval_s: float = 5.0, drop_grace_s: float = 30.0,
                 min_nodes: int = 1, store=None):
        self.topology = topology
        self.health_interval = health_interval_s
        self.drop_grace = drop_grace_s
        self.min_nodes = min_nodes
        self.phase = self.PHASE_RUNNING
        now = time.time()
        self._healths: Dict[int, _RankHealth] = {r: _RankHealth(r, now) for r in range(topology.world_size)}
        self._on_drop_callbacks: List[Callable[[List[int]], None]] = []
        self._store = store
        self._beat = 0
        self._seen: Dict[int, int] = {}

    def register_on_drop(self, cb: Callable[[List[int]], None]) -> None:
        self._on_drop_callbacks.append(cb)

    def _fire(self, dead: List[int]) -> None:
        for cb in self._on_drop_callbacks:
            try:
                cb(dead)
            except Exception:
                log.exception("on_drop callback failed")

    def _heartbeat_store(self) -> List[int]:
        self._beat += 1
        me = self.topology.rank
        self._store.set(f"hb/{me}", str(self._beat))
        now = time.time()
        dead: List[int] = []
        for r, h in self._healths.items():
            try:
                val = int(self._store.get(f"hb/{r}")) if r != me else self._beat
            except Exception:
                val = self._seen.get(r, 0)
            if val != self._seen.get(r):
                self._seen[r] = val
                h.last_heartbeat = now
                h.alive = True
            elif h.alive and (now - h.last_heartbeat) > self.drop_grace:
                h.alive = False
                dead.append(r)
        if dead:
            self._fire(dead)
        return dead

    def heartbeat(self) -> List[int]:
        """Probe the peers; returns the ranks that were newly declared dead."""
        if self.topology.world_size == 1:
            return []
        if self._store is not None:
            return self._heartbeat_store()
        if not dist.is_initialized():
            return []
        import datetime

        try:
            if hasattr(dist, "monitored_barrier") and dist.get_backend() == "gloo":
                dist.monitored_barrier(timeout=datetime.timedelta(seconds=self.drop_grace), wait_all_ranks=True)
            else:
                dist.barrier()
            now = time.time()
            for h in self._healths.values():
                h.last_heartbeat, h.alive = now, True
            return []
        except Exception as exc:
            log.warning("heartbeat barrier failed: %s", exc)
            now = time.time()
            dead = []
            for h in self._healths.values():
                if h.alive and (now - h.last_heartbeat) > self.drop_grace:
                    h.alive = False
                    dead.append(h.rank)
            if dead:
                self._fire(dead)
            return dead

    def mark_dead(self, ranks: List[int]) -> None:
        """Record an externally observed failure (e.g. the launcher reported the exit of a worker)."""
        newly = []
        for r in ranks:
            h = self._healths.get(r)
            if h is not None and h.alive:
                h.alive = False
                newly.append(r)
        if newly:
            self._fire(newly)

    def alive_ranks(self) -> List[int]:
        return [h.rank for h in self._healths.values() if h.alive]

    def begin_recovery(self) -> None:
        self.phase = self.PHASE_DRAINING

    def reshard(self, new_topology: ParallelTopology, num_experts: int) -> Dict[int, List[int]]:
        """``{ep_rank: [global expert ids]}`` for the new topology: contiguous blocks, remainder on the lowest ranks."""
        assignment = {r: new_topology.experts_on_rank(num_experts, r) for r in range(new_topology.ep_size)}
        self.phase = self.PHASE_RECOVERING
        return assignment

    def mark_resumed(self) -> None:
        self.phase = self.PHASE_RESUMED

    def _rebalance_experts(self, active_ranks: List[int], mesh, num_experts: int) -> Dict[int, List[int]]:
        """Round-robin spread of the experts over the surviving process ranks."""
        active = sorted(active_ranks)
        if not active:
            return {}
        out: Dict[int, List[int]] = {r: [] for r in active}
        for e in range(num_experts):
            out[active[e % len(active)]].append(e)
        return out

    def _on_rank_failure(self, dead_ranks: List[int]) -> None:
        log.warning("rank failure detected, dead=%s active=%s", dead_ranks, self.alive_ranks())


# ==================================================================================================
# harness
# ==================================================================================================
@dataclass
class ElasticConfig:
    local_ckpt_dir: str
    remote_uri: Optional[str]
    s3_endpoint: Optional[str] = None
    retention: int = 8
    async_workers: int = 4
    health_interval_s: float = 5.0
    drop_grace_s: float = 30.0
    min_nodes: int = 1


def _largest_divisor_le(n: int, k: int) -> int:
    """Largest d <= k that divides n (at least 1)."""
    d = max(1, min(k, n))
    while d > 1 and n % d != 0:
        d -= 1
    return d


class ElasticTrainerHarness:
    """Wires the checkpointer and the state machine together (``checkpoint``, ``health_check``, ``recover``)."""

    def __init__(self, cfg: ElasticConfig, topology: ParallelTopology, store=None):
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
        os.environ.setdefault("TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC", "30")
        os.environ.setdefault("TORCH_NCCL_TRACE_BUFFER_SIZE", "1048576")
        os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
        self.cfg, self.topology = cfg, topology
        self.rdzv_backend = os.environ.get("RDZV_BACKEND", "c10d")
        self.rdzv_epoch, self.rdzv_run_id = -1, ""
        if self.rdzv_backend == "etcd":
            self._init_etcd_rendezvous()
        self.local_adapter = LocalNVMeAdapter(cfg.local_ckpt_dir)
        self.remote_adapter: Optional[ObjectStoreAdapter] = None
        if cfg.remote_uri:
            if cfg.remote_uri.startswith("s3://") and _HAS_BOTO3:
                self.remote_adapter = S3Adapter(cfg.remote_uri, cfg.s3_endpoint)
            elif cfg.remote_uri.startswith("file://"):
                self.remote_adapter = LocalNVMeAdapter(cfg.remote_uri[len("file://"):], use_odirect=False)
        self.async_ckpt = AsyncCheckpointer(self.local_adapter, self.remote_adapter, retention=cfg.retention,
                                            workers=cfg.async_workers)
        self.state = ClusterStateMachine(topology, cfg.health_interval_s, cfg.drop_grace_s, cfg.min_nodes, store=store)
        self.state.register_on_drop(self.state._on_rank_failure)
        self._signals_installed = False
        self.last_reshard_plan: Optional[Dict[int, List[int]]] = None

    def _init_etcd_rendezvous(self) -> None:
        """Probe an etcd rendezvous (restart epoch tracking); any failure falls back to c10d."""
        try:
            from torch.distributed.elastic.rendezvous import etcd_rendezvous  # noqa: F401
        except Exception:
            log.warning("etcd rendezvous not available; falling back to c10d")
            self.rdzv_backend = "c10d"
            return
        self.rdzv_run_id = os.environ.get("RDZV_ID", "default-run")
        log.info("etcd rendezvous requested: run_id=%s endpoint=%s", self.rdzv_run_id,
                 os.environ.get("RDZV_ENDPOINT", "localhost:2379"))

    # ---- signals -----------------------------------------------------------------------------------
    def install_signal_handlers(self) -> None:
        if self._signals_installed:
            return
        for sig in (signal.SIGTERM, signal.SIGUSR1):
            try:
                signal.signal(sig, self._on_signal)
            except (ValueError, OSError):  # not the main thread
                pass
        self._signals_installed = True

    def _on_signal(self, signum, frame) -> None:
        log.warning("signal %d received; flushing the checkpoint queue", signum)
        self.async_ckpt.shutdown(drain=True)

    # ---- operations --------------------------------------------------------------------------------
    def checkpoint(self, model: torch.nn.Module, optimizer, step: int) -> None:
        self.async_ckpt.save(model, optimizer, step, rank=self.topology.rank, extra_meta={
            "dp_size": self.topology.dp_size, "ep_size": self.topology.ep_size, "tp_size": self.topology.tp_size,
            "pp_size": self.topology.pp_size, "world_size": self.topology.world_size,
            "ep_from_dp": self.topology.ep_from_dp})

    def health_check(self) -> List[int]:
        return self.state.heartbeat()

    def load_resharded(self, model: torch.nn.Module, step: int, old_meta: Dict[str, Any],
                       new_topo: ParallelTopology, num_experts: int) -> None:
        """Fill ``model`` (built for ``new_topo``) from files written under another expert-parallel degree.

        Dense parameters come from any old rank's file; the stacked expert weights (``*.w13`` / ``*.w2``) are
        assembled row by row from the old files that own the experts this rank holds now.
        """
        old_ep = int(old_meta.get("ep_size", 1))
        old_world = int(old_meta.get("world_size", 1))
        old_probe = ParallelTopology(old_world, 0, int(old_meta.get("dp_size", 1)), old_ep,
                                     int(old_meta.get("tp_size", 1)), int(old_meta.get("pp_size", 1)),
                                     ep_from_dp=bool(old_meta.get("ep_from_dp", False)))
        # one representative global rank per old ep rank
        rep: Dict[int, int] = {}
        for r in range(old_world):
            t = ParallelTopology(old_world, r, old_probe.dp_size, old_ep, old_probe.tp_size, old_probe.pp_size,
                                 ep_from_dp=old_probe.ep_from_dp)
            if t.tp_rank == new_topo.tp_rank and t.pp_rank == new_topo.pp_rank:
                rep.setdefault(t.ep_rank, r)
        cache: Dict[int, Dict[str, torch.Tensor]] = {}

        def old_model(ep_rank: int) -> Dict[str, torch.Tensor]:
            if ep_rank not in cache:
                cache[ep_rank] = self.async_ckpt.load_raw(step, rep[ep_rank])["model"]
            return cache[ep_rank]

        mine = new_topo.experts_on_this_rank(num_experts)
        sd = model.state_dict()
        base = old_model(min(rep))
        with torch.no_grad():
            for name, dst in sd.items():
                if name.rsplit(".", 1)[-1] in ("w13", "w2"):
                    for j, e in enumerate(mine):
                        owner = next(r for r in range(old_ep) if e in old_probe.experts_on_rank(num_experts, r))
                        local = old_probe.experts_on_rank(num_experts, owner).index(e)
                        dst[j].copy_(old_model(owner)[name][local])
                elif name in base:
                    dst.copy_(base[name])

    def recover(self, model: torch.nn.Module, optimizer, num_experts: int) -> ParallelTopology:
        """evict -> re-form the process group from the environment -> re-own experts -> reload -> resume."""
        log.warning("entering recovery on rank=%d", self.topology.rank)
        self.state.begin_recovery()
        if dist.is_initialized():
            dist.destroy_process_group()
        new_world = int(os.environ.get("WORLD_SIZE", str(self.topology.world_size)))
        new_rank = int(os.environ.get("RANK", str(self.topology.rank)))
        if new_world > 1:
            dist.init_process_group(backend="nccl" if torch.cuda.is_available() else "gloo", world_size=new_world,
                                    rank=new_rank)
        new_ep = _largest_divisor_le(new_world, self.topology.ep_size)
        new_dp = new_world // new_ep
        new_topo = build_topology(new_dp, new_ep, device_type=self.topology.device.type)
        self.state._rebalance_experts(self.state.alive_ranks(), self.topology.mesh, num_experts)
        self.last_reshard_plan = self.state.reshard(new_topo, num_experts)
        latest = self.async_ckpt.latest_step()
        if latest is not None:
            same_layout = (new_topo.ep_size == self.topology.ep_size and new_topo.world_size == self.topology.world_size)
            if same_layout:
                self.async_ckpt.load(model, optimizer, latest, rank=new_topo.rank)
            else:
                try:
                    meta = json.loads(self.local_adapter.get(
                        f"ckpts/step={latest:06d}/rank={0:06d}.meta.json").decode("utf-8"))
                except FileNotFoundError:
                    meta = {"ep_size": self.topology.ep_size, "dp_size": self.topology.dp_size,
                            "world_size": self.topology.world_size}
                try:
                    self.load_resharded(model, latest, meta, new_topo, num_experts)
                except Exception as exc:
                    log.warning("resharded load failed (%s); loading this rank's own file", exc)
                    self.async_ckpt.load(model, optimizer, latest, rank=new_topo.rank)
            log.info("resumed from step=%d on new topology dp=%d ep=%d", latest, new_dp, new_ep)
        else:
            log.warning("no checkpoint found; continuing from the current weights")
        self.state.mark_resumed()
        self.state.topology = new_topo
        self.topology = new_topo
        return new_topo

    def shutdown(self) -> None:
        self.async_ckpt.shutdown(drain=True)
