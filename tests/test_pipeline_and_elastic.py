"""Pipeline scheduling in one process, object stores, asynchronous checkpointer, state machine, harness
(reference: tests/test_pipeline_parallel.py, test_elastic.py, test_elastic_v02.py)."""

import json
import os
import threading
import time

import pytest
import torch
import torch.nn as nn

from composed_mixture_of_experts_engine_b200.elastic import (CHECKPOINT_SCHEMA_VERSION, AsyncCheckpointer,
                                                              ObjectStoreAdapter,
                                                             ClusterStateMachine, ElasticConfig,
                                                             ElasticTrainerHarness, LocalNVMeAdapter,
                                                             _check_schema_compatibility, _largest_divisor_le)
from composed_mixture_of_experts_engine_b200.parallel import ParallelTopology, PipelineStage, partition_layers

pytestmark = pytest.mark.cpu


# ---------------------------------------------------------------- pipeline
@pytest.mark.parametrize("p,m", [(1, 1), (2, 4), (4, 2), (4, 8), (3, 0)])
def test_run_1f1b_returns_one_grad_per_microbatch(p, m):
    stage = PipelineStage(0, p, module=nn.Linear(4, 4))
    mbs = [torch.randn(2, 4) for _ in range(m)]
    grads = stage.run_1f1b(mbs)
    assert len(grads) == m and all(g is not None and g.shape == (2, 4) for g in grads)


def test_stage_position_and_errors():
    s = PipelineStage(1, 3)
    assert not s.is_first and not s.is_last and PipelineStage(0, 3).is_first and PipelineStage(2, 3).is_last
    x = torch.randn(2, 2)
    assert torch.equal(s.forward_step(x), x) and torch.equal(s.backward_step(x), x)
    with pytest.raises(ValueError):
        PipelineStage(3, 3)
    with pytest.raises(RuntimeError):
        s.run_1f1b_distributed([x])


def test_partition_layers():
    assert [list(r) for r in partition_layers(10, 4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert sum(len(r) for r in partition_layers(32, 2)) == 32


# ---------------------------------------------------------------- object store
def test_local_adapter_round_trip_and_atomicity(tmp_path):
    st = LocalNVMeAdapter(str(tmp_path / "store"))
    st.put("ckpts/step=000001/rank=000000.pt", b"hello")
    st.put("ckpts/step=000001/rank=000000.meta.json", b"{}")
    assert st.get("ckpts/step=000001/rank=000000.pt") == b"hello"
    assert st.list("ckpts/") == ["ckpts/step=000001/rank=000000.meta.json", "ckpts/step=000001/rank=000000.pt"]
    assert st.list("nothing/") == []
    st.delete("ckpts/step=000001/rank=000000.pt")
    st.delete("ckpts/step=000001/rank=000000.pt")  # idempotent
    with pytest.raises(FileNotFoundError):
        st.get("ckpts/step=000001/rank=000000.pt")
    assert not list((tmp_path / "store").rglob("*.tmp"))


def test_local_adapter_large_unaligned_payload(tmp_path):
    st = LocalNVMeAdapter(str(tmp_path), chunk_bytes=1 << 20)
    payload = os.urandom(5 * (1 << 20) + 1234)  # several chunks and an unaligned tail
    st.put("big.bin", payload)
    assert st.get("big.bin") == payload
    st.put("empty.bin", b"")
    assert st.get("empty.bin") == b""


# ---------------------------------------------------------------- checkpointer
def _model_and_opt():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4))
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    m(torch.randn(3, 8)).sum().backward()
    opt.step()
    return m, opt


def test_save_load_bit_exact_and_meta(tmp_path):
    m, opt = _model_and_opt()
    ck = AsyncCheckpointer(LocalNVMeAdapter(str(tmp_path / "l")), LocalNVMeAdapter(str(tmp_path / "r")), workers=2)
    ck.save(m, opt, 7, rank=3, extra_meta={"dp_size": 2})
    ck.shutdown()
    assert ck.last_commit_ms >= 0 and ck.latest_step() == 7
    for tier in ("l", "r"):
        assert (tmp_path / tier / "ckpts" / "step=000007" / "rank=000003.pt").exists()
        meta = json.loads((tmp_path / tier / "ckpts" / "step=000007" / "rank=000003.meta.json").read_text())
        assert {"schema_version", "step", "rank", "hostname", "ts", "moe_engine_version", "torch_version",
                "dp_size"} <= set(meta)
        assert meta["schema_version"] == CHECKPOINT_SCHEMA_VERSION == 2
    m2, opt2 = _model_and_opt()
    with torch.no_grad():
        for p in m2.parameters():
            p.add_(1.0)
    ck2 = AsyncCheckpointer(LocalNVMeAdapter(str(tmp_path / "l")), None, workers=1)
    meta = ck2.load(m2, opt2, 7, rank=3)
    ck2.shutdown()
    assert meta["step"] == 7
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)
    s1, s2 = opt.state_dict()["state"], opt2.state_dict()["state"]
    assert all(torch.equal(s1[k]["exp_avg"], s2[k]["exp_avg"]) for k in s1)
    obj = torch.load(tmp_path / "l" / "ckpts" / "step=000007" / "rank=000003.pt", weights_only=False)
    assert set(obj) == {"model", "optim"} and {"state", "param_groups"} <= set(obj["optim"])


def test_retention_and_remote_fallback(tmp_path):
    m, opt = _model_and_opt()
    local, remote = LocalNVMeAdapter(str(tmp_path / "l")), LocalNVMeAdapter(str(tmp_path / "r"))
    ck = AsyncCheckpointer(local, remote, retention=2, workers=1)
    for s in range(1, 6):
        ck.save(m, opt, s)
    ck.shutdown()
    steps = {int(k.split("step=")[1][:6]) for k in local.list("ckpts/")}
    assert steps == {4, 5} and ck.latest_step() == 5
    # wipe the local tier: load falls back to the remote tier and re-hydrates the local one
    for k in local.list("ckpts/"):
        local.delete(k)
    m2, _ = _model_and_opt()
    ck2 = AsyncCheckpointer(local, remote, workers=1)
    ck2.load(m2, None, 5)
    ck2.shutdown()
    assert "ckpts/step=000005/rank=000000.pt" in local.list("ckpts/")


def test_pruning_never_deletes_a_newer_step_that_is_still_being_written(tmp_path):
    """Four writers, retention 1, a remote tier whose writes take a random few milliseconds: steps complete out of
    order, and a worker that finishes step s prunes while step s+1 is half written.  The newest step must survive
    in both tiers, and nothing older than the retained step may be left behind."""
    import random
    import time

    class Jittery(LocalNVMeAdapter):
        def put(self, key, payload):
            time.sleep(random.Random(hash(key) & 0xFFFF).random() * 0.02)
            super().put(key, payload)

        def put_torch(self, key, obj):
            time.sleep(random.Random(hash(key) & 0xFFFF).random() * 0.02)
            super().put_torch(key, obj)

    m, opt = _model_and_opt()
    local, remote = LocalNVMeAdapter(str(tmp_path / "l")), Jittery(str(tmp_path / "r"), use_odirect=False)
    ck = AsyncCheckpointer(local, remote, retention=1, workers=4)
    for s in range(1, 21):
        ck.save(m, opt, s)
    ck.shutdown()
    assert ck.last_error is None
    for store in (local, remote):
        keys = store.list("ckpts/")
        assert "ckpts/step=000020/rank=000000.pt" in keys and "ckpts/step=000020/rank=000000.meta.json" in keys
        assert all(int(k.split("step=")[1][:6]) >= 17 for k in keys)  # stragglers of in-flight saves at most
    m2, _ = _model_and_opt()
    ck2 = AsyncCheckpointer(local, remote, workers=1)
    assert ck2.latest_step() == 20
    ck2.load(m2, None, 20)
    ck2.shutdown()


def test_save_does_not_wait_for_slow_storage(tmp_path):
    class Slow(LocalNVMeAdapter):
        def put(self, key, payload):
            time.sleep(0.3)
            super().put(key, payload)

        def put_torch(self, key, obj):
            time.sleep(0.3)
            super().put_torch(key, obj)

    m, opt = _model_and_opt()
    ck = AsyncCheckpointer(Slow(str(tmp_path)), None, workers=1)
    t0 = time.perf_counter()
    ck.save(m, opt, 1)
    assert time.perf_counter() - t0 < 0.25  # enqueue only
    ck.shutdown(drain=True)
    assert ck.latest_step() == 1


def test_checkpoint_files_are_written_without_an_in_memory_copy(tmp_path):
    """The workers hand the snapshot itself to a local adapter (`put_torch`: torch's file writer, which does not
    hold the interpreter lock) and only small objects go through `put(bytes)`; an adapter without `put_torch`
    (an object store) still gets the serialised bytes."""
    seen = []

    class Spy(LocalNVMeAdapter):
        def put(self, key, payload):
            seen.append(("put", key, len(payload)))
            super().put(key, payload)

    class BytesOnly(ObjectStoreAdapter):
        """An adapter of the reference's interface only (what an object store offers)."""

        def __init__(self, root):
            self.inner = LocalNVMeAdapter(root, use_odirect=False)

        def put(self, key, payload):
            seen.append(("remote", key, len(payload)))
            self.inner.put(key, payload)

        def get(self, key):
            return self.inner.get(key)

        def list(self, prefix):
            return self.inner.list(prefix)

        def delete(self, key):
            self.inner.delete(key)

        def _p(self, key):
            return self.inner._p(key)

    m, opt = _model_and_opt()
    local, remote = Spy(str(tmp_path / "l")), BytesOnly(str(tmp_path / "r"))
    ck = AsyncCheckpointer(local, remote, workers=1)
    ck.save(m, opt, 3)
    ck.shutdown()
    assert ck.last_error is None
    assert [k for kind, k, _ in seen if kind == "put"] == ["ckpts/step=000003/rank=000000.meta.json"]
    assert ("ckpts/step=000003/rank=000000.pt" in [k for kind, k, _ in seen if kind == "remote"])
    for store in (local, remote):
        state = torch.load(store._p("ckpts/step=000003/rank=000000.pt"), map_location="cpu", weights_only=False)
        assert set(state) >= {"model"}
        for k, v in m.state_dict().items():
            assert torch.equal(state["model"][k], v)


def test_worker_survives_a_failing_store(tmp_path):
    class Flaky(LocalNVMeAdapter):
        n = 0

        def put(self, key, payload):
            Flaky.n += 1
            if Flaky.n == 1:
                raise OSError("injected storage failure")
            super().put(key, payload)

        def put_torch(self, key, obj):
            Flaky.n += 1
            if Flaky.n == 1:
                raise OSError("injected storage failure")
            super().put_torch(key, obj)

    m, opt = _model_and_opt()
    ck = AsyncCheckpointer(Flaky(str(tmp_path)), None, workers=1)
    ck.save(m, opt, 1)
    ck.save(m, opt, 2)
    ck.shutdown()
    assert isinstance(ck.last_error, OSError) and ck.latest_step() == 2


# ---------------------------------------------------------------- state machine / harness
def test_state_machine_phases_and_reshard():
    topo = ParallelTopology(world_size=8, rank=0, dp_size=1, ep_size=8)
    sm = ClusterStateMachine(topo)
    assert sm.phase == "running" and sm.heartbeat() == [] and sm.alive_ranks() == list(range(8))
    sm.begin_recovery()
    assert sm.phase == "draining"
    plan = sm.reshard(ParallelTopology(world_size=6, rank=0, dp_size=1, ep_size=6), 64)
    assert sm.phase == "recovering" and sorted(sum(plan.values(), [])) == list(range(64))
    assert [len(v) for v in plan.values()] == [11, 11, 11, 11, 10, 10]
    sm.mark_resumed()
    assert sm.phase == "resumed"
    rb = sm._rebalance_experts([5, 1, 3], None, 7)
    assert rb == {1: [0, 3, 6], 3: [1, 4], 5: [2, 5]} and sm._rebalance_experts([], None, 4) == {}


def test_store_heartbeat_detects_a_silent_rank():
    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v

        def get(self, k):
            return self[k]

    store = FakeStore()
    topo0 = ParallelTopology(world_size=2, rank=0, dp_size=2, ep_size=1)
    topo1 = ParallelTopology(world_size=2, rank=1, dp_size=2, ep_size=1)
    a = ClusterStateMachine(topo0, drop_grace_s=0.05, store=store)
    b = ClusterStateMachine(topo1, drop_grace_s=0.05, store=store)
    dropped = []
    a.register_on_drop(dropped.extend)
    b.heartbeat()
    assert a.heartbeat() == []
    time.sleep(0.08)  # rank 1 never beats again
    assert a.heartbeat() == [1] and dropped == [1] and a.alive_ranks() == [0]
    assert a.heartbeat() == []  # reported once
    a.mark_dead([0, 1])
    assert a.alive_ranks() == []


@pytest.mark.parametrize("n,k,want", [(8, 8, 8), (6, 8, 6), (6, 4, 3), (7, 4, 1), (12, 5, 4), (1, 8, 1)])
def test_largest_divisor(n, k, want):
    assert _largest_divisor_le(n, k) == want


def test_schema_check_never_raises():
    for v in (1, 2, 3):
        _check_schema_compatibility({"schema_version": v})
    _check_schema_compatibility({})


def test_harness_checkpoint_meta_and_signal_handlers_from_thread(tmp_path):
    topo = ParallelTopology(world_size=1, rank=0, dp_size=1, ep_size=1)
    h = ElasticTrainerHarness(ElasticConfig(str(tmp_path / "l"), "file://" + str(tmp_path / "r"), async_workers=1), topo)
    err = []
    t = threading.Thread(target=lambda: (h.install_signal_handlers(), err.append(None)))
    t.start()
    t.join()
    assert err == [None]
    m, opt = _model_and_opt()
    h.checkpoint(m, opt, 3)
    assert h.health_check() == []
    h.shutdown()
    meta = json.loads((tmp_path / "r" / "ckpts" / "step=000003" / "rank=000000.meta.json").read_text())
    assert meta["dp_size"] == 1 and meta["ep_size"] == 1 and meta["world_size"] == 1


def test_resharded_load_re_owns_experts(tmp_path):
    """Files written under ep=2 are loaded into an ep=1 model: every expert row comes from its old owner."""
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer

    torch.manual_seed(0)
    full = DistributedMoELayer(8, 16, 4, 2)
    store = LocalNVMeAdapter(str(tmp_path / "l"))
    ck = AsyncCheckpointer(store, None, workers=1)
    for r in range(2):
        topo = ParallelTopology(world_size=2, rank=r, dp_size=1, ep_size=2)
        part = DistributedMoELayer(8, 16, 4, 2, topology=topo)
        with torch.no_grad():
            part.w13.copy_(full.w13[2 * r:2 * r + 2])
            part.w2.copy_(full.w2[2 * r:2 * r + 2])
            part.router.gate_w.copy_(full.router.gate_w)
        ck.save(part, None, 9, rank=r, extra_meta={"ep_size": 2, "dp_size": 1, "world_size": 2})
    ck.shutdown()
    new_topo = ParallelTopology(world_size=1, rank=0, dp_size=1, ep_size=1)
    h = ElasticTrainerHarness(ElasticConfig(str(tmp_path / "l"), None, async_workers=1), new_topo)
    fresh = DistributedMoELayer(8, 16, 4, 2)
    h.load_resharded(fresh, 9, {"ep_size": 2, "dp_size": 1, "world_size": 2}, new_topo, 4)
    h.shutdown()
    assert torch.equal(fresh.w13, full.w13) and torch.equal(fresh.w2, full.w2)
    assert torch.equal(fresh.router.gate_w, full.router.gate_w)


def test_generation_store_is_private_to_the_restart(monkeypatch):
    """Without a TorchElastic launcher there is nothing to prefix; with one, the keys of two restart generations do
    not see each other (a restarted worker must not read addresses its dead predecessor's peers published)."""
    import torch.distributed as dist

    from composed_mixture_of_experts_engine_b200.engine import elastic_generation_store
    from tests.conftest import find_free_port

    for var in ("TORCHELASTIC_RESTART_COUNT", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_USE_AGENT_STORE"):
        monkeypatch.delenv(var, raising=False)
    assert elastic_generation_store(0, 1) is None
    port = find_free_port()
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(port))
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "0")
    gen0 = elastic_generation_store(0, 1)  # rank 0 hosts the store when the launcher does not
    assert isinstance(gen0, dist.PrefixStore)
    gen0.set("addr", "old")
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "1")
    monkeypatch.setenv("TORCHELASTIC_USE_AGENT_STORE", "True")  # second generation: connect as a client
    gen1 = elastic_generation_store(0, 1)
    assert gen1.num_keys() >= 1 and not gen1.check(["addr"])
    gen1.set("addr", "new")
    assert gen0.get("addr") == b"old" and gen1.get("addr") == b"new"


class _FakeS3Client:
    """In-memory stand-in for the four boto3 calls the S3 tier makes."""

    def __init__(self):
        self.objects = {}

    def put_object(self, Bucket, Key, Body):
        self.objects[(Bucket, Key)] = bytes(Body)

    def get_object(self, Bucket, Key):
        import io

        if (Bucket, Key) not in self.objects:
            raise KeyError(Key)
        return {"Body": io.BytesIO(self.objects[(Bucket, Key)])}

    def delete_object(self, Bucket, Key):
        self.objects.pop((Bucket, Key), None)

    def get_paginator(self, name):
        assert name == "list_objects_v2"
        client = self

        class _Pages:
            def paginate(self, Bucket, Prefix):
                keys = sorted(k for (b, k) in client.objects if b == Bucket and k.startswith(Prefix))
                for i in range(0, max(len(keys), 1), 2):  # two keys per page: the adapter must walk all pages
                    yield {"Contents": [{"Key": k} for k in keys[i:i + 2]]} if keys else {}

        return _Pages()


def test_s3_tier_with_a_stand_in_client(monkeypatch, tmp_path):
    """Remote tier on S3 (reference: LocalNVMeAdapter + S3Adapter, pkg/elastic/fault_monitor.py:220-259): keys carry
    the URI's prefix, listing walks every page and strips the prefix, and a checkpoint that only survives remotely is
    loaded from there and written back to the local tier."""
    import types

    import torch

    from composed_mixture_of_experts_engine_b200.elastic import fault_monitor as fm

    fake = _FakeS3Client()
    monkeypatch.setattr(fm, "_HAS_BOTO3", True)
    monkeypatch.setattr(fm, "boto3", types.SimpleNamespace(client=lambda *a, **k: fake), raising=False)
    monkeypatch.setattr(fm, "BotoConfig", lambda **k: None, raising=False)
    with pytest.raises(ValueError):
        fm.S3Adapter("file:///tmp/x")
    s3 = fm.S3Adapter("s3://bucket/run-7/")
    for i in range(5):
        s3.put(f"ckpts/step={i:06d}/rank=000000.pt", b"x%d" % i)
    assert ("bucket", "run-7/ckpts/step=000003/rank=000000.pt") in fake.objects
    assert s3.list("ckpts/") == [f"ckpts/step={i:06d}/rank=000000.pt" for i in range(5)]
    assert s3.get("ckpts/step=000004/rank=000000.pt") == b"x4"
    s3.delete("ckpts/step=000004/rank=000000.pt")
    assert len(s3.list("ckpts/")) == 4

    model = torch.nn.Linear(8, 8)
    ck = fm.AsyncCheckpointer(fm.LocalNVMeAdapter(str(tmp_path / "local")), fm.S3Adapter("s3://bucket/run-8"), workers=1)
    ck.save(model, None, 3)
    ck.shutdown(drain=True)
    assert any(k.startswith("run-8/ckpts/step=000003/") for (_, k) in fake.objects)
    # the local tier is lost; a fresh checkpointer finds the step remotely and restores it locally
    import shutil

    shutil.rmtree(tmp_path / "local")
    other = torch.nn.Linear(8, 8)
    ck2 = fm.AsyncCheckpointer(fm.LocalNVMeAdapter(str(tmp_path / "local")), fm.S3Adapter("s3://bucket/run-8"), workers=1)
    ck2.load(other, None, 3)
    ck2.shutdown(drain=True)
    assert all(torch.equal(a, b) for a, b in zip(model.parameters(), other.parameters()))
    assert list((tmp_path / "local").rglob("*.pt"))
