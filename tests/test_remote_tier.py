"""Remote tier on CPU: block-addressed files and the key-addressed store, write-through on
put, three-fragment get, prefetch, host-side fault injection (reference: tests/test_mooncake_*.py)."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.external.remote_store import FaultInjector, KVStoreBackend, LoopbackKVStore
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def start(cache_kw):
    shape = KVShape("r", 2, 2, 16, tokens_per_block=T)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=24, **cache_kw),
                    require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=5)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    return mgr, kv


@pytest.mark.parametrize("kind", ["files", "kvstore"])
def test_remote_write_through_and_restore(tmp_path, kind, monkeypatch):
    kw = dict(enable_remote=True, num_remote_blocks=64)
    if kind == "files":
        kw.update(remote_cache_path=str(tmp_path), remote_file_num=3)
    else:
        kw.update(use_mooncake_store_backend=True, mooncake_store_config_path="loopback",
                  remote_config_custom={"store": LoopbackKVStore()})
    mgr, kv = start(kw)
    try:
        tok = np.arange(8 * T, dtype=np.int64)
        src = np.array([3, 9, 1, 30, 12, 7, 50, 2])
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        saved = [t.clone() for t in kv]
        mgr._clear_cpu_cache()                       # only the remote tier still has the blocks
        for t in kv:
            t.zero_()
        tid, mask = mgr.get_match(tok)
        if kind == "kvstore":
            # a store behind a network is never read on the compute path: the get misses (the engine recomputes
            # or has prefetched); tests/test_mooncake_prefetch_compute_split.py in the reference pins the same
            assert int(mask.sum()) == 0
            mgr.cancel(tid)
            monkeypatch.setenv("FLEXKV_REMOTE_STORE_IN_GRAPH", "1")     # engines without a prefetch hook
            mgr.kv_task_engine.cache_engine._store_in_graph = True
            tid, mask = mgr.get_match(tok)
        assert int(mask.sum()) == 8 * T
        kinds = sorted(o.transfer_type.value for o in mgr.kv_task_engine.tasks[tid].graph.ops())
        assert kinds == ["H2D", "REMOTE2H"]
        dst = np.arange(40, 48)
        mgr.launch(tid, slots(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], saved[l][:, src])
        # the pulled blocks were adopted by the host tier: the next get is host-only
        tid, mask = mgr.get_match(tok)
        assert [o.transfer_type.value for o in mgr.kv_task_engine.tasks[tid].graph.ops()] == ["H2D"]
        mgr.cancel(tid)
        # prefetch pulls remote blocks into the host pool ahead of time (from either kind of remote tier,
        # whatever the compute-path rule says)
        mgr.kv_task_engine.cache_engine._store_in_graph = False
        mgr._clear_cpu_cache()
        pid = mgr.prefetch_async(tok)
        r = mgr.wait(pid, completely=True)[pid]
        assert r.status.value == "success" and int(r.return_mask.sum()) == 8 * T
        tid, mask = mgr.get_match(tok, cpu_only=True)
        assert int(mask.sum()) == 8 * T
        mgr.cancel(tid)
        tid, mask = mgr.get_match(tok)               # and the compute-path get now hits the host tier
        assert int(mask.sum()) == 8 * T
        assert [o.transfer_type.value for o in mgr.kv_task_engine.tasks[tid].graph.ops()] == ["H2D"]
        mgr.cancel(tid)
    finally:
        mgr.shutdown()


def test_injected_remote_failure_fails_the_get_and_rolls_back(monkeypatch):
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_MODE", "tail")
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_OP", "get")
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_TAIL_N", "2")
    monkeypatch.setenv("FLEXKV_REMOTE_STORE_IN_GRAPH", "1")     # the get itself reads the store in this test
    mgr, kv = start(dict(enable_remote=True, use_mooncake_store_backend=True, mooncake_store_config_path="loopback",
                         remote_config_custom={"store": LoopbackKVStore()}))
    try:
        tok = np.arange(6 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots(range(6)))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        mgr._clear_cpu_cache()
        tid = mgr.get_async(tok, slots(range(10, 16)))
        assert mgr.wait(tid, timeout=5)[tid].status.value == "failed"       # two tail blocks did not arrive
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        assert cpu.mempool.num_used_blocks == 0 and cpu.index.is_empty()    # staging returned, nothing adopted
    finally:
        mgr.shutdown()


def test_fault_injector_modes():
    assert FaultInjector("none").apply("get", [True, True]) == [True, True]
    assert FaultInjector("all").apply("get", [True, True]) == [False, False]
    assert FaultInjector("tail", tail_n=1).apply("put", [True, True, True]) == [True, True, False]
    assert FaultInjector("tail", op="get").apply("put", [True, True]) == [True, True]
    r = FaultInjector("random", seed=1, random_ratio=0.5).apply("get", [True] * 8)
    assert r.count(False) == 4
    s = KVStoreBackend(LoopbackKVStore())
    blk = np.arange(16, dtype=np.uint8)
    assert s.put([7, 8], [blk, blk]) == [True, True] and s.prefix_hit(np.array([7, 8, 9], dtype=np.uint64)) == 2


def test_prefetch_reports_the_longest_prefix_that_arrived(monkeypatch):
    """Per-block failures injected on the host: a prefetch keeps the blocks before the first failure."""
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_MODE", "tail")
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_OP", "get")
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_TAIL_N", "2")
    mgr, kv = start(dict(enable_remote=True, use_mooncake_store_backend=True, mooncake_store_config_path="loopback",
                         remote_config_custom={"store": LoopbackKVStore()}))
    try:
        tok = np.arange(6 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots(range(6)))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        saved = [t.clone() for t in kv]
        mgr._clear_cpu_cache()
        pid = mgr.prefetch_async(tok)
        r = mgr.wait(pid, completely=True)[pid]
        assert r.status.value == "success" and int(r.return_mask.sum()) == 4 * T      # 6 asked, last 2 failed
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        assert cpu.mempool.num_used_blocks == 4
        # the adopted prefix serves a host-only get with the right bytes
        tid, mask = mgr.get_match(tok, cpu_only=True)
        assert int(mask.sum()) == 4 * T
        mgr.launch(tid, slots(range(20, 24)))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, 20:24], saved[l][:, 0:4])
    finally:
        mgr.shutdown()


def test_a_key_addressed_store_needs_a_connector_that_prefetches(monkeypatch):
    from flexkv_b200.common.config import assert_mooncake_prefetch_ready
    monkeypatch.delenv("FLEXKV_REMOTE_STORE_IN_GRAPH", raising=False)
    store = CacheConfig(enable_remote=True, use_mooncake_store_backend=True)
    assert_mooncake_prefetch_ready(store, prefetch_enabled=True)
    assert_mooncake_prefetch_ready(CacheConfig(), prefetch_enabled=False)        # no store: nothing to gate
    with pytest.raises(RuntimeError, match="prefetch"):
        assert_mooncake_prefetch_ready(store, prefetch_enabled=False)
    monkeypatch.setenv("FLEXKV_REMOTE_STORE_IN_GRAPH", "1")
    assert_mooncake_prefetch_ready(store, prefetch_enabled=False)


@pytest.mark.parametrize("kind", ["files", "kvstore"])
def test_a_put_that_is_local_already_retries_the_upload_the_remote_tier_misses(tmp_path, kind, monkeypatch):
    """First put: the upload fails (host-side fault injection), the local tiers keep the blocks. Second put of the
    same tokens: nothing to copy from the GPU, but the remote tier still misses the blocks, so the plan is one
    H2REMOTE fed by the ready host blocks (reference: tests/test_mooncake_deferred_put.py
    test_ready_cpu_hit_retries_a_missing_mooncake_upload_without_d2h)."""
    kw = dict(enable_remote=True, num_remote_blocks=64)
    if kind == "files":
        kw.update(remote_cache_path=str(tmp_path), remote_file_num=2)
    else:
        kw.update(use_mooncake_store_backend=True, remote_config_custom={"store": LoopbackKVStore()})
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_MODE", "all")
    monkeypatch.setenv("FLEXKV_MOONCAKE_FAULT_OP", "put")
    mgr, kv = start(kw)
    try:
        tok = np.arange(5 * T, dtype=np.int64) + 4242
        src = np.array([3, 9, 1, 30, 12])
        tid = mgr.put_async(tok, slots(src))
        r = mgr.wait(tid, completely=True)[tid]              # the GPU->host part ended; the upload failed
        gce = mgr.kv_task_engine.cache_engine
        from flexkv_b200.common.block import SequenceMeta
        seq = SequenceMeta(tok, T)
        assert gce.cpu_cache_engine.match(seq).num_ready_matched_blocks == 5
        assert gce._remote_lacks(seq, 5)
        # the store works again
        backend = gce.remote_backend or mgr.kv_task_engine.transfer_handles[0].engine._workers[
            next(k for k in mgr.kv_task_engine.transfer_handles[0].engine._workers
                 if getattr(k[1], "value", k[1]) == "H2REMOTE")].backend
        backend.fault.mode = "none"
        tid, mask = mgr.put_match(tok)
        ops = [o.transfer_type.value for o in mgr.kv_task_engine.tasks[tid].graph.ops()]
        assert ops == ["H2REMOTE"], ops
        assert int(mask.sum()) == 0                          # no GPU block is read
        mgr.launch(tid, slots(src)[:0])
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert not gce._remote_lacks(seq, 5)
        tid, mask = mgr.put_match(tok)                       # now there is nothing left to do
        assert mgr.kv_task_engine.tasks[tid].graph.num_ops == 0
        mgr.cancel(tid)
        # and the uploaded bytes are the real ones
        saved = [t.clone() for t in kv]
        mgr._clear_cpu_cache()
        pid = mgr.prefetch_async(tok)
        assert int(mgr.wait(pid, completely=True)[pid].return_mask.sum()) == 5 * T
        tid, mask = mgr.get_match(tok)
        mgr.launch(tid, slots(np.arange(40, 45)))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, 40:45], saved[l][:, src])
    finally:
        mgr.shutdown()
