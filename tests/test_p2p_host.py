"""Two nodes of one box share prefixes through the registry: node B restores blocks that
only node A's host pool holds (PEERH2H), node liveness, stale-node cleanup and the
registry served over ZeroMQ (reference flow: flexkv/cache/hie_cache_engine.py:239-334,
flexkv/cache/redis_meta.py:296-430,514-617; worker flexkv/transfer/worker.py:2920-3029)."""
import time
import uuid

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.cache.registry import (NodeRegistry, RegistryClient, RegistryMetaChannel, RegistryServer,
                                        RegistryStore)
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def start_node(name, seed):
    shape = KVShape("p", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=24, enable_p2p_cpu=True, redis_host=f"inproc:{name}")
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=seed)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    return mgr, kv


def test_node_b_restores_from_node_a_host_pool():
    name = uuid.uuid4().hex
    a, kva = start_node(name, 1)
    b, kvb = start_node(name, 2)
    try:
        ea = a.kv_task_engine.cache_engine.cpu_cache_engine
        eb = b.kv_task_engine.cache_engine.cpu_cache_engine
        assert ea.node_id != eb.node_id
        tok = np.arange(10 * T, dtype=np.int64) + 1000
        src = np.array([5, 6, 7, 20, 21, 3, 40, 41, 42, 43])
        tid = a.put_async(tok, slots(src))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        # B already holds the first 3 blocks itself (different bytes do not matter: same tokens)
        for l in range(2):
            kvb[l][:, src[:3]] = kva[l][:, src[:3]]
        tid = b.put_async(tok[:3 * T], slots(src[:3]))
        assert b.wait(tid, completely=True)[tid].status.value == "success"
        ea.refresh(); eb.refresh()
        from flexkv_b200.common.block import SequenceMeta
        local, remote, winner = eb.match_all(SequenceMeta(tok, T))
        assert winner == "remote" and remote.num_matched_blocks == 10 and local.num_ready_matched_blocks == 3
        assert set(remote.node_ids.tolist()) == {ea.node_id}

        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 10 * T
        kinds = sorted(o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops())
        assert kinds == ["H2D", "PEERH2H"]
        dst = np.arange(50, 60)
        for t in kvb:
            t[:, dst] = 0
        b.launch(tid, slots(dst))
        assert b.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kvb[l][:, dst], kva[l][:, src])
        # the pulled blocks were adopted by B's host tier: the next get needs no peer
        tid, mask = b.get_match(tok)
        assert [o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops()] == ["H2D"]
        b.cancel(tid)
    finally:
        a.shutdown()
        b.shutdown()


def test_peer_that_left_is_not_offered_and_a_vanished_pool_fails_cleanly():
    name = uuid.uuid4().hex
    a, kva = start_node(name, 1)
    b, kvb = start_node(name, 2)
    try:
        ea = a.kv_task_engine.cache_engine.cpu_cache_engine
        eb = b.kv_task_engine.cache_engine.cpu_cache_engine
        tok = np.arange(6 * T, dtype=np.int64) + 5000
        tid = a.put_async(tok, slots(range(6)))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        ea.refresh(); eb.refresh()
        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 6 * T
        # the owner's pool disappears between planning and the copy (host-side fault): the op
        # fails per block, the get reports failure and B's staging blocks return to its pool
        w = next(w for (k, tt), w in b.transfer_manager.engine._workers.items() if tt.value == "PEERH2H")
        real = w.registry.get_node_meta
        w.registry.get_node_meta = lambda nid, pp_rank=None: {}
        free_before = eb.mempool.num_free_blocks
        b.launch(tid, slots(range(30, 36)))
        r = b.wait(tid)[tid]
        assert r.status.value == "failed"
        w.registry.get_node_meta = real
        assert eb.mempool.num_free_blocks == free_before + 6
        # A leaves the box: its records are withdrawn and B stops offering them
        a.shutdown()
        eb.refresh()
        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 0
        b.cancel(tid)
    finally:
        a.shutdown()
        b.shutdown()


def test_registry_liveness_and_stale_cleanup_with_a_fake_clock():
    now = [1000.0]
    store = RegistryStore(clock=lambda: now[0])
    c = RegistryClient(store)
    n1 = NodeRegistry(c, ip="10.0.0.1", node_ttl_seconds=5, instance_uuid="u1")
    n2 = NodeRegistry(c, ip="10.0.0.2", node_ttl_seconds=5, instance_uuid="u2")
    id1, id2 = n1.register(), n2.register()
    assert (id1, id2) == (1, 2) and n1.active_nodes() == [1, 2]
    ch = RegistryMetaChannel(c)
    ch.publish(id1, [(0, 7, id1, 0xABC, 99999, 0)])
    n1.set_node_meta(dict(pool_file="/dev/shm/x", block_bytes=4096, num_blocks=8))
    assert n2.get_node_meta(id1)["pool_file"] == "/dev/shm/x"
    assert store.scan("CPUB:block:1:") == ["CPUB:block:1:0000000000000abc"]
    now[0] += 4
    assert c.expire(f"node:{id2}", 5)              # node 2 heartbeats, node 1 does not
    now[0] += 2
    assert n2.active_nodes() == [2] and ch.list_nodes() == [2]
    assert not c.expire(f"node:{id1}", 5)          # an expired node is not resurrected
    # the same instance registers again: new id, old records swept
    c.hset(f"node:{id1}", dict(node_id=id1, ip="10.0.0.1", uuid="u1", status="active"))
    id1b = n1.register()
    assert id1b == 3 and store.scan("CPUB:block:1:") == [] and n1.active_nodes() == [2, 3]
    # reset barrier: both live nodes must acknowledge
    assert not n1.reset_barrier(1, timeout=0.05)
    n2.client.hset("reset:1", {str(id2): 1})
    assert n1.reset_barrier(1, timeout=0.5)


def test_registry_over_zeromq(tmp_path):
    pytest.importorskip("zmq")
    ep = f"ipc://{tmp_path}/reg.sock"
    srv = RegistryServer(ep)
    try:
        c1, c2 = RegistryClient(ep), RegistryClient(ep)
        assert c1.incr("global:node_id") == 1 and c2.incr("global:node_id") == 2
        c1.hset("node:1", dict(node_id=1, status="active"), ttl=0.2)
        assert c2.hgetall("node:1")["status"] == "active"
        ch = RegistryMetaChannel(c1)
        ch.publish(1, [(0, 1, 1, 11, 5000, 0), (11, 2, 1, 12, 5000, 0)])
        assert sorted(r[3] for r in RegistryMetaChannel(c2).load(1)) == [11, 12]
        time.sleep(0.3)
        assert c2.hgetall("node:1") == {}
        with pytest.raises(RuntimeError):
            c1._call("no_such_command")
    finally:
        srv.close()


def test_node_b_restores_from_node_a_ssd_files(tmp_path):
    """A prefix that node A holds only on SSD (its host pool is too small to keep it) is read by node B out of
    A's block files (PEERSSD2H), staged in B's host pool and restored (reference: PEER2CPUTransferWorker's
    peer-SSD path, flexkv/transfer/worker.py:2920-3873; planner flexkv/cache/cache_engine.py:2963-3060)."""
    name = uuid.uuid4().hex
    shape = KVShape("p", 2, 2, 16, tokens_per_block=T)

    def start(seed, sub, cpu_blocks):
        cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=cpu_blocks, enable_ssd=True, num_ssd_blocks=64,
                          ssd_cache_dir=str(tmp_path / sub), enable_p2p_cpu=True, enable_p2p_ssd=True,
                          redis_host=f"inproc:{name}")
        mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
        kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=seed)
        mgr.register_gpu_tensors(kv, layout)
        mgr.start(); mgr.wait_ready(30)
        return mgr, kv

    a, kva = start(1, "a", 12)
    b, kvb = start(2, "b", 24)
    try:
        ga, gb = a.kv_task_engine.cache_engine, b.kv_task_engine.cache_engine
        tok = np.arange(10 * T, dtype=np.int64) + 7000
        src = np.array([5, 6, 7, 20, 21, 3, 40, 41, 42, 43])
        tid = a.put_async(tok, slots(src))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        # push the prefix out of A's 12-block host pool: only the SSD tier keeps it
        other = np.arange(10 * T, dtype=np.int64) + 90000
        tid = a.put_async(other, slots(np.arange(50, 60)))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        from flexkv_b200.common.block import SequenceMeta
        seq = SequenceMeta(tok, T)
        assert ga.cpu_cache_engine.match(seq).num_ready_matched_blocks < 10
        assert ga.ssd_cache_engine.match(seq).num_ready_matched_blocks == 10
        for e in (ga.cpu_cache_engine, ga.ssd_cache_engine, gb.cpu_cache_engine, gb.ssd_cache_engine):
            e.refresh()
        assert gb.ssd_cache_engine.match_remote(seq).num_matched_blocks == 10
        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 10 * T
        kinds = sorted(o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops())
        assert "PEERSSD2H" in kinds and "H2D" in kinds, kinds
        dst = np.arange(20, 30)
        for t in kvb:
            t[:, dst] = 0
        b.launch(tid, slots(dst))
        assert b.wait(tid, timeout=30)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kvb[l][:, dst], kva[l][:, src])
        # adopted by B's host tier: the next get is local
        tid, mask = b.get_match(tok)
        assert [o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops()] == ["H2D"]
        b.cancel(tid)
    finally:
        a.shutdown()
        b.shutdown()


def test_cluster_wide_reset_withdraws_every_nodes_blocks():
    """Both nodes reset at the same time: each drops its blocks, withdraws its published records and returns
    once the other has acknowledged the same epoch; afterwards neither finds the old prefix anywhere
    (reference: tests/test_hierarchy_reset.py, flexkv/cache/hie_cache_engine.py:177-223)."""
    import threading
    name = uuid.uuid4().hex
    a, kva = start_node(name, 1)
    b, kvb = start_node(name, 2)
    try:
        ea = a.kv_task_engine.cache_engine.cpu_cache_engine
        eb = b.kv_task_engine.cache_engine.cpu_cache_engine
        tok = np.arange(6 * T, dtype=np.int64) + 300
        tid = a.put_async(tok, slots([1, 2, 3, 4, 5, 6]))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        ea.refresh(); eb.refresh()
        assert int(b.get_match(tok)[1].sum()) == 6 * T
        t0 = time.monotonic()
        ths = [threading.Thread(target=m.reset) for m in (a, b)]
        for t in ths:
            t.start()
        for t in ths:
            t.join(30)
        assert time.monotonic() - t0 < 10, "the reset barrier ran into its timeout"
        ea.refresh(); eb.refresh()
        assert int(a.get_match(tok)[1].sum()) == 0 and int(b.get_match(tok)[1].sum()) == 0
        assert ea.channel.load(ea.node_id) == [] and eb.match_remote(
            __import__("flexkv_b200.common.block", fromlist=["SequenceMeta"]).SequenceMeta(tok, T)).num_matched_blocks == 0
        # the tiers work again afterwards
        tid = b.put_async(tok, slots([7, 8, 9, 10, 11, 12]))
        assert b.wait(tid, completely=True)[tid].status.value == "success"
        eb.refresh(); ea.refresh()                          # B publishes, then A rebuilds its view
        assert int(a.get_match(tok)[1].sum()) == 6 * T
    finally:
        a.shutdown()
        b.shutdown()


def test_node_b_restores_from_the_files_node_a_wrote_to_the_shared_remote_mount(tmp_path):
    """enable_3rd_remote: every node writes remote files of its own on a mount all nodes see and publishes which
    blocks they hold; node B, which never saw the prompt, reads the blocks out of A's files (REMOTE2H with owner
    ids), adopts them into its host tier and restores them (the role PCFS has in the reference:
    flexkv/cache/hie_cache_engine.py:239-378,561-643; tests/test_pcfs*.py need its SDK)."""
    import os
    name = uuid.uuid4().hex
    shape = KVShape("p", 2, 2, 16, tokens_per_block=T)
    shared = tmp_path / "mount"

    def start(seed, cpu_blocks):
        cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=cpu_blocks, enable_remote=True, enable_3rd_remote=True,
                          num_remote_blocks=64, remote_cache_path=str(shared), remote_file_num=2,
                          remote_file_prefix="kv", redis_host=f"inproc:{name}")
        mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
        kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=seed)
        mgr.register_gpu_tensors(kv, layout)
        mgr.start(); mgr.wait_ready(30)
        return mgr, kv

    a, kva = start(1, 12)
    b, kvb = start(2, 24)
    try:
        ga, gb = a.kv_task_engine.cache_engine, b.kv_task_engine.cache_engine
        names = sorted(os.listdir(shared))
        assert len(names) == 4 and len({n.rsplit("_", 1)[0] for n in names}) == 2, names   # two files per node
        tok = np.arange(10 * T, dtype=np.int64) + 7000
        src = np.array([5, 6, 7, 20, 21, 3, 40, 41, 42, 43])
        tid = a.put_async(tok, slots(src))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        # push the prefix out of A's 12-block host pool: only its remote files keep it
        other = np.arange(10 * T, dtype=np.int64) + 90000
        tid = a.put_async(other, slots(np.arange(50, 60)))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        from flexkv_b200.common.block import SequenceMeta
        seq = SequenceMeta(tok, T)
        assert ga.cpu_cache_engine.match(seq).num_ready_matched_blocks < 10
        assert ga.remote_cache_engine.match(seq).num_ready_matched_blocks == 10
        ga.remote_cache_engine.refresh(); gb.remote_cache_engine.refresh()
        assert gb.remote_cache_engine.match_remote(seq).num_matched_blocks == 10
        assert gb.remote_cache_engine.match(seq).num_matched_blocks == 0           # B itself holds nothing
        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 10 * T
        ops = list(b.kv_task_engine.tasks[tid].graph.ops())
        kinds = sorted(o.transfer_type.value for o in ops)
        assert kinds == ["H2D", "REMOTE2H"], kinds
        assert next(o for o in ops if o.transfer_type.value == "REMOTE2H").remote_node_ids is not None
        dst = np.arange(20, 30)
        for t in kvb:
            t[:, dst] = 0
        b.launch(tid, slots(dst))
        assert b.wait(tid, timeout=30)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kvb[l][:, dst], kva[l][:, src])
        # adopted by B's host tier: the next get is local
        tid, mask = b.get_match(tok)
        assert [o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops()] == ["H2D"]
        b.cancel(tid)
        # an owner whose files are gone fails the op, it does not hang or return stale bytes
        tok2 = np.arange(4 * T, dtype=np.int64) + 555000
        tid = a.put_async(tok2, slots(np.array([1, 2, 3, 4])))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        ga.remote_cache_engine.refresh(); gb.remote_cache_engine.refresh()
        w = next(w for (k, tt), w in b.kv_task_engine.transfer_handles[0].engine._workers.items()
                 if getattr(tt, "value", tt) == "REMOTE2H")
        w.close()
        meta_key_files = [str(shared / n) for n in names]
        a_id = ga.node_registry.node_id
        hidden = [f for f in meta_key_files if f"_n{a_id}_" in f]
        for f in hidden:
            os.rename(f, f + ".gone")
        # A still serves its host copy to itself; B has to go through A's files, which are gone
        tid, mask = b.get_match(tok2)
        assert int(mask.sum()) == 4 * T
        b.launch(tid, slots(np.arange(30, 34)))
        assert b.wait(tid, timeout=30)[tid].status.value == "failed"
        for f in hidden:
            os.rename(f + ".gone", f)
    finally:
        a.shutdown()
        b.shutdown()


def test_registry_inspector_lists_nodes_metadata_and_block_records():
    """`benchmarks/registry_check.py` against the registry of a two-node deployment (in-process store here; the same
    calls go to a RegistryServer or a Redis server): both nodes alive, their pool files in the metadata, the
    publisher's host blocks counted."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "registry_check", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks",
                                       "registry_check.py"))
    rc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rc)
    from flexkv_b200.cache.registry import connect
    name = uuid.uuid4().hex
    a, kva = start_node(name, 1)
    b, kvb = start_node(name, 2)
    try:
        tok = np.arange(6 * T, dtype=np.int64) + 4100
        tid = a.put_async(tok, slots([1, 2, 3, 4, 5, 6]))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        a.kv_task_engine.cache_engine.cpu_cache_engine.refresh()
        report = rc.inspect(connect(f"inproc:{name}", 0))
        assert [n["alive"] for n in report["nodes"]] == [True, True]
        by_id = {n["node_id"]: n for n in report["nodes"]}
        aid = a.kv_task_engine.cache_engine.node_registry.node_id
        assert by_id[aid]["blocks"]["host"]["records"] == 6 and len(by_id[aid]["blocks"]["host"]["sample"]) == 2
        assert sum(n["blocks"]["host"]["records"] for n in report["nodes"]) == 6
        assert any("pool_file" in m for n in report["nodes"] for m in n["meta"].values())
        assert report["records_of_unknown_nodes"] == {}
        text = rc.render(report)
        assert f"node {aid}: alive" in text and "host: 6 block records" in text
    finally:
        a.shutdown()
        b.shutdown()
