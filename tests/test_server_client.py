"""Server-client mode on CPU: two data-parallel KVManager front ends share one
index through the ZeroMQ server; GPU tensors (host stand-ins here) arrive as
handles over the registration socket (reference: tests/test_kvmanager_client_api.py,
test_external_server_mode.py, test_registration_key.py)."""
import os
import time

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager, KVTPClient
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
from flexkv_b200.common.memory_handle import alloc_shared_host_tensor
from flexkv_b200.server.utils import unique_ipc_endpoint


def slots(blocks, T):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def test_two_dp_ranks_share_one_server():
    shape = KVShape("s", 2, 2, 16, tokens_per_block=4)
    T = 4
    model = make_model_config(shape, dp_size=2)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    ep, reg = unique_ipc_endpoint("srv"), unique_ipc_endpoint("reg")
    m0 = KVManager(model, cache, dp_client_id=0, server_recv_port=ep, gpu_register_port=reg, require_gpu=True)
    m1 = KVManager(model, cache, dp_client_id=1, server_recv_port=ep, gpu_register_port=reg)
    assert m0.server_client_mode and m0.server_handle is not None and m1.server_handle is None
    caches = []
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=70 + d)
        KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout, mode="same_process")
        caches.append(kv)
    m0.start(); m1.start()
    try:
        m0.wait_ready(30); m1.wait_ready(30)
        tok = np.arange(6 * T, dtype=np.int64)
        src = np.array([3, 9, 1, 30, 12, 7])
        tid = m0.put_async(tok, slots(src, T))
        assert m0.wait(tid, completely=True)[tid].status.value == "success"
        # the other rank sees the prefix and restores it into its own cache
        tid, mask = m1.get_match(tok)
        assert int(mask.sum()) == 6 * T
        dst = np.array([0, 1, 2, 3, 4, 5])
        assert m1.launch(tid, slots(dst, T)) == [tid]
        assert m1.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(caches[1][l][:, dst], caches[0][l][:, src])
        assert m1.try_wait(tid)[tid].status.value == "not_found"
        m1.reset()
        assert int(m0.get_match(tok)[1].sum()) == 0
        with pytest.raises(RuntimeError):
            m0.launch(12345, slots(dst, T))        # server-side errors come back as exceptions
        # a client that leaves gives back what it had reserved; the server keeps serving the other one
        tid = m0.put_async(tok, slots(src, T))
        assert m0.wait(tid, completely=True)[tid].status.value == "success"
        pending, mask = m1.get_match(tok)
        assert int(mask.sum()) == 6 * T
        assert m1.dp_client.unregister() == 1
        assert m1.dp_client.unregister() == 0                      # already gone
        assert int(m0.get_match(tok)[1].sum()) == 6 * T
        assert m1.is_ready()                                       # registers again on its next call
    finally:
        m1.shutdown(); m0.shutdown()


def test_tp_client_sleep_and_wake_over_the_registration_channel():
    """An engine worker asks the data plane to let go of its tensors, re-creates them and
    re-registers; a get issued while asleep completes into the new tensors."""
    shape = KVShape("s", 2, 2, 16, tokens_per_block=4)
    T = 4
    model = make_model_config(shape, dp_size=2)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    ep, reg = unique_ipc_endpoint("srv"), unique_ipc_endpoint("reg")
    m0 = KVManager(model, cache, dp_client_id=0, server_recv_port=ep, gpu_register_port=reg, require_gpu=True)
    m1 = KVManager(model, cache, dp_client_id=1, server_recv_port=ep, gpu_register_port=reg)
    clients, caches = [], []
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=90 + d)
        c = KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0)
        c.register_to_server(kv, layout, mode="same_process")
        clients.append(c); caches.append((kv, layout))
    m0.start(); m1.start()
    try:
        m0.wait_ready(30); m1.wait_ready(30)
        tok = np.arange(4 * T, dtype=np.int64) + 40
        tid = m0.put_async(tok, slots([5, 6, 7, 8], T))
        assert m0.wait(tid, completely=True)[tid].status.value == "success"
        want = [t[:, 5:9].clone() for t in caches[0][0]]
        assert clients[1].suspend_gpu_mappings(timeout=10)
        tid = m1.get_async(tok, slots([20, 21, 22, 23], T))
        time.sleep(0.2)
        assert m1.wait(tid, timeout=0.2)[tid].status.value != "success"          # parked
        tid0 = m0.put_async(tok + 1000, slots([1, 2, 3, 4], T))                  # the other client is unaffected
        assert m0.wait(tid0, completely=True)[tid0].status.value == "success"
        kv2, layout2 = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="zeros")
        assert clients[1].resume_gpu_mappings(kv2, layout2, mode="same_process")
        assert m1.wait(tid, timeout=10)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv2[l][:, 20:24], want[l])
    finally:
        for c in clients:
            c.shutdown()
        m1.shutdown(); m0.shutdown()


def test_external_server_process(tmp_path, monkeypatch):
    """The server runs as its own process; the manager only creates clients."""
    import json
    import subprocess
    import sys
    from flexkv_b200.common.config import GLOBAL_CONFIG_FROM_ENV
    T = 4
    shape = KVShape("x", 2, 2, 16, tokens_per_block=T)
    ep, reg = unique_ipc_endpoint("xsrv"), unique_ipc_endpoint("xreg")
    mcfg = dict(num_layers=2, num_kv_heads=2, head_size=16, dtype="bfloat16", dp_size=2)
    ccfg = dict(tokens_per_block=T, num_cpu_blocks=16)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, "-m", "flexkv_b200.server", "--model-config", json.dumps(mcfg),
                             "--cache-config", json.dumps(ccfg), "--recv-endpoint", ep, "--gpu-register-port", reg,
                             "--no-gpu"], cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    monkeypatch.setattr(GLOBAL_CONFIG_FROM_ENV, "server_launch_mode", "external")
    mgrs, tp_clients = [], []
    t0 = time.time()
    while not os.path.exists(reg[len("ipc://"):]) and time.time() - t0 < 60:      # the server binds its sockets
        time.sleep(0.1)
    try:
        model = make_model_config(shape, dp_size=2)
        cache = CacheConfig(**ccfg)
        keep = []
        for d in range(2):
            mgrs.append(KVManager(model, cache, dp_client_id=d, server_recv_port=ep, gpu_register_port=reg))
            assert mgrs[-1].server_handle is None
            src_kv, layout = alloc_paged_cache(shape, 16, "cpu", "vllm", fill="normal", seed=d)
            # another process cannot open host stand-ins by address: put them in shared files
            kv = []
            for i, t in enumerate(src_kv):
                s = alloc_shared_host_tensor(t.shape, t.dtype, str(tmp_path / f"kv_{d}_{i}.bin"))
                s.copy_(t)
                kv.append(s)
            tp_clients.append(KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0))
            tp_clients[-1].register_to_server(kv, layout)
            keep.append(kv)
        for m in mgrs:
            m.start()
        for m in mgrs:
            m.wait_ready(60)
        tok = np.arange(3 * T, dtype=np.int64)
        tid = mgrs[0].put_async(tok, slots([1, 2, 3], T))
        assert mgrs[0].wait(tid, completely=True)[tid].status.value == "success"
        tid = mgrs[1].get_async(tok, slots([5, 6, 7], T))
        assert mgrs[1].wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(keep[1][l][:, 5:8], keep[0][l][:, 1:4])
    finally:
        for m in mgrs:
            m.shutdown()
        proc.terminate()
        try:
            out, _ = proc.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
    assert proc.returncode in (0, -15), out[-2000:]


def test_batch_launch_over_the_server_returns_per_request_masks():
    """The flow of the throughput benchmark in server-client mode: several matches, one batched
    launch, one wait on the batch id whose response lists a mask per request."""
    shape = KVShape("s", 2, 2, 16, tokens_per_block=4)
    T = 4
    model = make_model_config(shape, dp_size=2)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    ep, reg = unique_ipc_endpoint("srv"), unique_ipc_endpoint("reg")
    m0 = KVManager(model, cache, dp_client_id=0, server_recv_port=ep, gpu_register_port=reg, require_gpu=True)
    m1 = KVManager(model, cache, dp_client_id=1, server_recv_port=ep, gpu_register_port=reg)
    caches = []
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=90 + d)
        KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout, mode="same_process")
        caches.append(kv)
    m0.start(); m1.start()
    try:
        m0.wait_ready(30); m1.wait_ready(30)
        rng = np.random.default_rng(3)
        for d, m in enumerate((m0, m1)):
            toks = [rng.integers(0, 1000, size=3 * T, dtype=np.int64) for _ in range(3)]
            src = rng.permutation(32)[:9].reshape(3, 3)
            ids = [m.put_match(t)[0] for t in toks]
            bid = m.launch(ids, [slots(b, T) for b in src], as_batch=True)
            res = m.wait(bid, timeout=30, completely=True)
            assert [r.status.value for r in res.values()] == ["success"]
            masks = next(iter(res.values())).return_mask
            assert isinstance(masks, list) and [int(x.sum()) for x in masks] == [3 * T] * 3
            dst = np.setdiff1d(np.arange(32), src.ravel())[:9].reshape(3, 3)
            ids = []
            for t in toks:
                tid, mask = m.get_match(t)
                assert int(mask.sum()) == 3 * T
                ids.append(tid)
            bid = m.launch(ids, [slots(b, T) for b in dst], as_batch=True)
            res = m.wait(bid, timeout=30)
            assert [r.status.value for r in res.values()] == ["success"]
            for l in range(2):
                assert torch.equal(caches[d][l][:, dst.ravel()], caches[d][l][:, src.ravel()])
    finally:
        m1.shutdown(); m0.shutdown()


def test_blocking_wait_of_one_client_does_not_hold_up_the_others():
    """The server parks a blocking wait and keeps serving: while rank 0 waits for a slow offload, rank 1's
    requests are answered at once (one loop serves every data-parallel rank)."""
    import threading
    from flexkv_b200.common.transfer import TransferType, WorkerKey
    shape = KVShape("s", 2, 2, 16, tokens_per_block=4)
    T = 4
    model = make_model_config(shape, dp_size=2)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    ep, reg = unique_ipc_endpoint("srv"), unique_ipc_endpoint("reg")
    m0 = KVManager(model, cache, dp_client_id=0, server_recv_port=ep, gpu_register_port=reg, require_gpu=True)
    m1 = KVManager(model, cache, dp_client_id=1, server_recv_port=ep, gpu_register_port=reg)
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=50 + d)
        KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout, mode="same_process")
    m0.start(); m1.start()
    try:
        m0.wait_ready(30); m1.wait_ready(30)
        w = m0.server_handle.server.transfer_manager.engine.worker_for(WorkerKey(0, 0), TransferType.D2H)
        plain = w.execute

        def slow(op):
            time.sleep(0.8)
            return plain(op)
        w.execute = slow
        tok = np.arange(4 * T, dtype=np.int64)
        got = {}

        def offload():
            tid = m0.put_async(tok, slots([1, 2, 3, 4], T))
            got["rsp"] = m0.wait(tid, timeout=30, completely=True)[tid]
            got["t"] = time.monotonic()
        th = threading.Thread(target=offload)
        t0 = time.monotonic()
        th.start()
        time.sleep(0.1)                                   # rank 0 is inside its wait now
        for i in range(5):
            tid, mask = m1.get_match(np.arange(100 + i, 100 + i + 2 * T, dtype=np.int64))
            assert int(mask.sum()) == 0
        served = time.monotonic() - t0
        th.join(30)
        assert got["rsp"].status.value == "success"
        assert served < 0.6 < got["t"] - t0, (served, got["t"] - t0)
        # a wait whose time runs out answers TIMEOUT and leaves the task waitable
        tid = m0.put_async(np.arange(500, 500 + 2 * T, dtype=np.int64), slots([9, 10], T))
        assert m0.wait(tid, timeout=0.2, completely=True)[tid].status.value == "timeout"
        assert m0.wait(tid, timeout=30, completely=True)[tid].status.value == "success"
    finally:
        m1.shutdown(); m0.shutdown()


def test_server_sleeps_on_requests_and_completions_not_on_a_timer():
    """While a client waits, the server's loop sleeps until a request or a completion arrives (the data plane's
    completion queue is a pollable descriptor); completions nobody waits for do not make it spin."""
    from flexkv_b200 import _native
    s = _native.C.GraphScheduler()
    fd = s.completion_fd()
    assert fd >= 0 and s.completion_fd() == fd
    import select
    assert select.select([fd], [], [], 0)[0] == []
    s.submit(1, [1], [0], [])
    s.op_done(1, 1, True, 0.1, 8)
    assert select.select([fd], [], [], 1.0)[0] == [fd]          # readable while records are waiting
    assert len(s.wait(0.0)) == 2
    assert select.select([fd], [], [], 0)[0] == []              # and quiet again once they were taken

    shape = KVShape("s", 2, 2, 16, tokens_per_block=4)
    T = 4
    model = make_model_config(shape, dp_size=2)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    ep, reg = unique_ipc_endpoint("srvfd"), unique_ipc_endpoint("regfd")
    m0 = KVManager(model, cache, dp_client_id=0, server_recv_port=ep, gpu_register_port=reg, require_gpu=True)
    m1 = KVManager(model, cache, dp_client_id=1, server_recv_port=ep, gpu_register_port=reg)
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=7 + d)
        KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout, mode="same_process")
    m0.start(); m1.start()
    try:
        m0.wait_ready(30); m1.wait_ready(30)
        srv = m0.server_handle.server
        lat = []
        for i in range(30):
            tok = np.arange(6 * T, dtype=np.int64) + 1000 * i
            tid = m0.put_async(tok, slots([1, 2, 3, 4, 5, 6], T))
            t0 = time.perf_counter()
            assert m0.wait(tid, completely=True)[tid].status.value == "success"
            lat.append(time.perf_counter() - t0)
        assert srv._completion_fds, "the server never found a descriptor to poll"
        assert sorted(lat)[len(lat) // 2] < 0.05
        # puts that nobody waits for: their completions must not leave the loop spinning
        for i in range(5):
            m1.put_async(np.arange(6 * T, dtype=np.int64) + 777000 + 1000 * i, slots([7, 8, 9, 10, 11, 12], T))
        time.sleep(0.3)
        c0 = time.process_time()
        time.sleep(0.5)
        assert time.process_time() - c0 < 0.4, "an idle server burns CPU"       # a spinning loop would use the whole 0.5 s
    finally:
        m1.shutdown()
        m0.shutdown()
