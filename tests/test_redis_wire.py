"""The registry over the Redis wire protocol: native RESP client, the registry's command set on top of it,
node registry and block-record channel against a Redis stand-in
(reference: csrc/dist/redis_meta_channel.cpp:60-215, flexkv/cache/redis_meta.py:158-906,
tests/test_redis_meta.py)."""
import time

import pytest

from flexkv_b200 import _native
from flexkv_b200.cache.redis_client import RedisRegistryClient
from flexkv_b200.cache.registry import NodeRegistry, RegistryMetaChannel, RegistryStore, connect
from fake_redis import FakeRedis

C = _native.C


@pytest.fixture
def server():
    s = FakeRedis()
    yield s
    s.stop()


def test_wire_encoding_and_incremental_parsing():
    assert C.RespClient.encode("HSET", "k", b"\x00\r\n") == b"*3\r\n$4\r\nHSET\r\n$1\r\nk\r\n$3\r\n\x00\r\n\r\n"
    reply = b"*4\r\n:7\r\n$-1\r\n*2\r\n+OK\r\n$5\r\nab\r\nc\r\n$0\r\n\r\n"
    for cut in range(len(reply)):
        assert C.RespClient.parse(reply[:cut]) is None              # incomplete: nothing consumed
    val, used = C.RespClient.parse(reply + b":1\r\n")
    assert used == len(reply) and val == [7, None, ["OK", b"ab\r\nc"], b""]
    with pytest.raises(RuntimeError, match="WRONGTYPE"):
        C.RespClient.parse(b"-WRONGTYPE nope\r\n")


def test_commands_agree_with_the_in_process_store(server):
    r = RedisRegistryClient("127.0.0.1", server.port)
    s = RegistryStore()
    assert r.ping()
    for c in (r, s):
        assert [c.incr("global:node_id") for _ in range(3)] == [1, 2, 3]
        assert c.hset("node:1", dict(node_id=1, ip="10.0.0.1", status="active", timestamp=12.5), ttl=5.0)
        assert not c.hset("node:9", dict(x=1), only_if_exists=True)
        assert c.hset("node:1", dict(status="draining"), only_if_exists=True)
        assert c.hgetall("node:1") == dict(node_id=1, ip="10.0.0.1", status="draining", timestamp=12.5)
        assert c.hgetall("nope") == {}
        assert c.exists("node:1") and not c.exists("node:2")
        assert c.expire("node:1", 5.0) and not c.expire("node:2", 5.0)
        n = c.hset_many([(f"CPUB:block:1:{i:016x}", dict(ph=i, pb=i + 1, nid=1, hash=2**63 + i, lt=-5, state=0))
                         for i in range(40)])
        assert n == 40
        assert len(c.scan("CPUB:block:1:")) == 40 and c.scan("CPUB:block:2:") == []      # several SCAN pages
        rows = c.scan_values("CPUB:block:1:")
        assert sorted(x["hash"] for x in rows) == [2**63 + i for i in range(40)] and rows[0]["lt"] == -5
        assert c.delete([f"CPUB:block:1:{i:016x}" for i in range(3)] + ["absent"]) == 3
        assert c.delete_prefix("CPUB:block:1:") == 37
        assert c.scan("") == ["node:1"] if c is s else "node:1" in c.scan("")
    assert "SCAN" in server.store.commands and "PEXPIRE" in server.store.commands


def test_node_registry_and_block_channel_over_redis(server):
    a = NodeRegistry(connect("redis://127.0.0.1", server.port), ip="10.0.0.1", node_ttl_seconds=0.4,
                     heartbeat_interval=0.05)
    b = NodeRegistry(connect(f"redis://127.0.0.1:{server.port}/0", 0), ip="10.0.0.2", node_ttl_seconds=0.4,
                     heartbeat_interval=0.05)
    na, nb = a.register(), b.register()
    assert (na, nb) == (1, 2)
    a.start_heartbeat()                                   # only a keeps its key alive
    a.set_node_meta(dict(pool_file="/dev/shm/pool_a", block_bytes=4096, num_blocks=128))
    assert b.get_node_meta(na) == dict(pool_file="/dev/shm/pool_a", block_bytes=4096, num_blocks=128, pp_rank=0,
                                       pp_size=1)
    ch = RegistryMetaChannel(a.client)
    ch.publish(na, [(11, 0, na, 0xFFFFFFFFFFFFFF01, 99, 0), (0xFFFFFFFFFFFFFF01, 1, na, 12, 99, 1)])
    ch.publish(nb, [(5, 3, nb, 77, 99, 0)])
    assert ch.list_nodes() == [na, nb]
    assert sorted(ch.load(na)) == sorted([(11, 0, na, 0xFFFFFFFFFFFFFF01, 99, 0), (0xFFFFFFFFFFFFFF01, 1, na, 12, 99, 1)])
    ch.remove(na, [12])
    assert [r[3] for r in ch.load(na)] == [0xFFFFFFFFFFFFFF01]
    time.sleep(0.7)                                       # b never renewed: it drops out, a stays
    assert ch.list_nodes() == [na] and a.active_nodes() == [na]
    assert not b.client.expire(f"node:{nb}", 1.0)         # and cannot be resurrected
    # the native tree publishes through the same channel
    ch.clear_node(na)
    assert ch.load(na) == []
    a.stop()
    assert a.client.scan("node:") == []


def test_broken_connection_is_an_error_then_reconnects(server):
    r = RedisRegistryClient("127.0.0.1", server.port, timeout_ms=500)
    assert r.incr("c") == 1
    server.drop_next = True
    with pytest.raises(ConnectionError):
        r.incr("c")
    assert r.incr("c") == 2                               # a fresh connection
    with pytest.raises(RuntimeError, match="unknown command"):
        r._c.command("FLUSHALL")
    dead = RedisRegistryClient("127.0.0.1", 1, timeout_ms=200)
    with pytest.raises(ConnectionError):
        dead.ping()


def test_password_and_database_are_sent_on_connect():
    s = FakeRedis(password="s3cret")
    try:
        ok = connect("redis://:s3cret@127.0.0.1/2", s.port)
        assert ok.incr("k") == 1
        assert s.store.commands[:2] == ["AUTH", "SELECT"]
        assert connect("redis://127.0.0.1", s.port, password="s3cret").incr("k") == 2     # CacheConfig.redis_password
        with pytest.raises(ConnectionError, match="AUTH refused"):
            RedisRegistryClient("127.0.0.1", s.port, password="wrong").ping()
    finally:
        s.stop()


def test_native_channel_and_python_channel_read_each_other(server):
    """Block records written from native code and from Python share one schema in the server."""
    cl = connect("redis://127.0.0.1", server.port)
    cl.hset("node:1", dict(node_id=1, status="active"), ttl=30)
    cl.hset("node:2", dict(node_id=2, status="left"), ttl=30)
    cl.hset("node:3", dict(node_id=3, status="active"), ttl=30)
    py_ch = RegistryMetaChannel(cl)
    nat = cl.native_channel("CPUB")
    rows = [(0, 5, 1, 2**64 - 7, -3, 0), (2**64 - 7, 6, 1, 1234567, 99, 1)] + \
           [(i, i, 1, 10_000 + i, 5, 0) for i in range(30)]                       # several SCAN pages
    nat.publish(1, rows)
    py_ch.publish(3, [(1, 2, 3, 4, 5, 2)])
    assert nat.list_nodes() == [1, 3] == py_ch.list_nodes()
    assert sorted(nat.load(1)) == sorted(rows) == sorted(py_ch.load(1))
    assert nat.load(3) == [(1, 2, 3, 4, 5, 2)]
    nat.remove(1, [1234567, 10_003])
    assert len(py_ch.load(1)) == 30 and (2**64 - 7, 6, 1, 1234567, 99, 1) not in py_ch.load(1)
    nat.clear_node(1)
    assert nat.load(1) == [] and py_ch.load(3) == [(1, 2, 3, 4, 5, 2)]
    server.drop_next = True
    with pytest.raises(ConnectionError):
        nat.list_nodes()
    assert nat.list_nodes() == [1, 3]


def test_two_nodes_share_prefixes_through_a_redis_registry(server):
    """The cross-node reuse flow of tests/test_p2p_host.py with the registry in a Redis server: node ids,
    liveness, node meta and block records all travel over the wire protocol, the block records from native code."""
    import numpy as np
    import torch
    from flexkv_b200 import CacheConfig, KVManager
    from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
    T = 4

    def slots(blocks):
        return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))

    def start(seed):
        shape = KVShape("p", 2, 2, 16, tokens_per_block=T)
        cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=24, enable_p2p_cpu=True, redis_host="redis://127.0.0.1",
                          redis_port=server.port)
        mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
        kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=seed)
        mgr.register_gpu_tensors(kv, layout)
        mgr.start(); mgr.wait_ready(30)
        return mgr, kv

    a, kva = start(1)
    b, kvb = start(2)
    try:
        ea = a.kv_task_engine.cache_engine.cpu_cache_engine
        eb = b.kv_task_engine.cache_engine.cpu_cache_engine
        assert type(ea.channel).__name__ == "RedisMetaChannel" and {ea.node_id, eb.node_id} == {1, 2}
        tok = np.arange(6 * T, dtype=np.int64) + 500
        src = np.array([5, 6, 7, 20, 21, 3])
        tid = a.put_async(tok, slots(src))
        assert a.wait(tid, completely=True)[tid].status.value == "success"
        ea.refresh(); eb.refresh()
        assert any(k.startswith(b"CPUB:block:") for k in server.store.d)
        # the registry inspector reads the same deployment over the wire protocol
        import importlib.util
        import os
        spec = importlib.util.spec_from_file_location("registry_check", os.path.join(
            os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "registry_check.py"))
        rc = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(rc)
        from flexkv_b200.cache.registry import connect
        report = rc.inspect(connect("redis://127.0.0.1", server.port))
        assert [n["node_id"] for n in report["nodes"]] == [1, 2] and all(n["alive"] for n in report["nodes"])
        assert {n["node_id"]: n["blocks"]["host"]["records"] for n in report["nodes"]} == {ea.node_id: 6, eb.node_id: 0}
        tid, mask = b.get_match(tok)
        assert int(mask.sum()) == 6 * T
        assert sorted(o.transfer_type.value for o in b.kv_task_engine.tasks[tid].graph.ops()) == ["H2D", "PEERH2H"]
        dst = np.arange(40, 46)
        b.launch(tid, slots(dst))
        assert b.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kvb[l][:, dst], kva[l][:, src])
    finally:
        a.shutdown()
        b.shutdown()
    assert not any(k.startswith(b"node:") for k in server.store.d)          # both left the registry
