"""Sliding-window snapshots end to end on the CPU tier: a put mounts the window page of the
sequence end on the new host node, a window-aware get is gated to the deepest snapshot and
restores full KV plus the page, snapshots are evicted LRU-first when the pool is full
(reference behaviour: flexkv/cache/swa_cache_engine.py:142-239, tests/test_swa_control_plane_e2e.py)."""
import numpy as np
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.common.config import SWAPoolConfig
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
from flexkv_b200.swa import SWAHostPool

T = 4
SWA_LAYERS, PAGE_BYTES = 3, 64


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def start(num_slots=4, device="cpu"):
    shape = KVShape("s", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_swa_transfer=True,
                      swa=SWAPoolConfig(enabled=True, num_slots=num_slots, num_swa_layers=SWA_LAYERS,
                                        bytes_per_token_per_layer=PAGE_BYTES // T, evict_ratio=0.25))
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    dev = "cpu" if device == "cpu" else torch.device(device)
    kv, layout = alloc_paged_cache(shape, 64, dev, "vllm", fill="normal", seed=5)
    mgr.register_gpu_tensors(kv, layout)
    g = torch.Generator().manual_seed(9)
    swa = [torch.randint(0, 256, (16, PAGE_BYTES), dtype=torch.uint8, generator=g).to(dev) for _ in range(SWA_LAYERS)]
    mgr.register_swa_tensors(swa)
    mgr.start(); mgr.wait_ready(30)
    return mgr, kv, swa


def put(mgr, tok, blocks, page):
    tid, mask = mgr.put_match(tok)
    mgr.launch(tid, slots(blocks)[mask[:len(blocks) * T]] if mask.any() else slots(blocks)[:0],
               swa_slot_mappings=[slots([page])])
    return mgr.wait(tid, completely=True)[tid]


import pytest


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_put_mounts_and_window_aware_get_restores_page_and_blocks(device):
    mgr, kv, swa = start(device=device)
    try:
        tok = np.arange(6 * T, dtype=np.int64) + 100
        src = np.array([3, 9, 1, 30, 12, 7])
        assert put(mgr, tok, src, page=5).status.value == "success"
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        assert cpu.index.total_swa_slots() == 1 and cpu.swa_pool.num_used == 1
        want_page = [t[5].clone() for t in swa]
        want_kv = [t[:, src].clone() for t in kv]
        # a longer query still only resumes at the snapshot (6 blocks), and a shorter one finds nothing
        long_tok = np.concatenate([tok, np.arange(2 * T) + 9000])
        tid, mask = mgr.get_match(long_tok, swa_aware=True)
        assert int(mask.sum()) == 6 * T
        kinds = sorted((o.transfer_type.value, o.is_swa) for o in mgr.kv_task_engine.tasks[tid].graph.ops()
                       if o.transfer_type.value != "Virtual")
        assert kinds == [("H2D", False), ("H2D", True)]
        dst = np.arange(40, 46)
        for t in swa:
            t[11] = 0
        mgr.launch(tid, slots(dst), swa_slot_mappings=[slots([11])])
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], want_kv[l])
        for l in range(SWA_LAYERS):
            assert torch.equal(swa[l][11], want_page[l])
        tid, mask = mgr.get_match(tok[:4 * T], swa_aware=True)
        assert int(mask.sum()) == 0
        mgr.cancel(tid)
        # without window awareness the plain prefix match is unchanged
        tid, mask = mgr.get_match(tok[:4 * T])
        assert int(mask.sum()) == 4 * T
        mgr.cancel(tid)
        # the node stays window-locked only while the get runs
        m = cpu.match(__import__("flexkv_b200.common.block", fromlist=["SequenceMeta"]).SequenceMeta(tok, T))
        assert cpu.index.swa_lock_cnt(m.last_swa_node) == 0
    finally:
        mgr.shutdown()


def test_launch_without_window_pages_drops_the_side_ops_and_returns_the_slot():
    mgr, kv, swa = start()
    try:
        tok = np.arange(3 * T, dtype=np.int64) + 500
        tid, mask = mgr.put_match(tok)
        mgr.launch(tid, slots([1, 2, 3]))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        assert cpu.index.total_swa_slots() == 0 and cpu.swa_pool.num_used == 0
        tid = mgr.put_async(tok + 1, slots([4, 5, 6]))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert cpu.swa_pool.num_used == 0
    finally:
        mgr.shutdown()


def test_full_pool_evicts_least_recently_used_snapshots():
    mgr, kv, swa = start(num_slots=2)
    try:
        cpu = mgr.kv_task_engine.cache_engine.cpu_cache_engine
        seqs = [np.arange(2 * T, dtype=np.int64) + 1000 * (i + 1) for i in range(3)]
        for i, tok in enumerate(seqs):
            assert put(mgr, tok, [2 * i, 2 * i + 1], page=i).status.value == "success"
        assert cpu.swa_pool.num_used <= 2 and cpu.index.total_swa_slots() == cpu.swa_pool.num_used
        # the oldest sequence lost its snapshot (an unlocked leaf goes with its blocks)
        tid, mask = mgr.get_match(seqs[0], swa_aware=True)
        assert int(mask.sum()) == 0
        mgr.cancel(tid)
        tid, mask = mgr.get_match(seqs[2], swa_aware=True)
        assert int(mask.sum()) == 2 * T
        mgr.cancel(tid)
    finally:
        mgr.shutdown()


def test_slot_pool():
    p = SWAHostPool(SWAPoolConfig(enabled=True, num_slots=3))
    a, b, c = p.allocate(), p.allocate(), p.allocate()
    assert (a, b, c) == (0, 1, 2) and p.allocate() is None and p.num_used == 3
    p.free(b); p.free(b)
    assert p.num_free == 1 and p.allocate() == 1
    p.reset()
    assert p.num_free == 3


def start_tiered(tmp_path, num_slots=4, num_ssd_slots=8, device="cpu"):
    shape = KVShape("s", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=64,
                      ssd_cache_dir=str(tmp_path), enable_swa_transfer=True,
                      swa=SWAPoolConfig(enabled=True, num_slots=num_slots, num_ssd_slots=num_ssd_slots,
                                        num_swa_layers=SWA_LAYERS, bytes_per_token_per_layer=PAGE_BYTES // T,
                                        evict_ratio=0.25))
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    dev = "cpu" if device == "cpu" else torch.device(device)
    kv, layout = alloc_paged_cache(shape, 64, dev, "vllm", fill="normal", seed=5)
    mgr.register_gpu_tensors(kv, layout)
    g = torch.Generator().manual_seed(9)
    swa = [torch.randint(0, 256, (16, PAGE_BYTES), dtype=torch.uint8, generator=g).to(dev) for _ in range(SWA_LAYERS)]
    mgr.register_swa_tensors(swa)
    mgr.start(); mgr.wait_ready(30)
    return mgr, kv, swa


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_ssd_window_tier_serves_the_snapshot_after_the_host_copy_is_gone(tmp_path, device):
    """A put writes the window page through to the SSD window file and mounts it on the SSD node; once the
    host tier has lost the sequence, a window-aware get reads full KV and the page back from SSD."""
    mgr, kv, swa = start_tiered(tmp_path, device=device)
    try:
        gce = mgr.kv_task_engine.cache_engine
        cpu, ssd = gce.cpu_cache_engine, gce.ssd_cache_engine
        tok = np.arange(5 * T, dtype=np.int64) + 700
        src = np.array([3, 9, 1, 30, 12])
        tid, mask = mgr.put_match(tok)
        kinds = sorted((o.transfer_type.value, o.is_swa) for o in mgr.kv_task_engine.tasks[tid].graph.ops()
                       if o.transfer_type.value != "Virtual")
        assert kinds == [("D2H", False), ("D2H", True), ("H2DISK", False), ("H2DISK", True)]
        mgr.launch(tid, slots(src), swa_slot_mappings=[slots([5])])
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert cpu.index.total_swa_slots() == 1 and ssd.index.total_swa_slots() == 1
        assert cpu.swa_pool.num_used == 1 and ssd.swa_pool.num_used == 1
        want_page = [t[5].clone() for t in swa]
        want_kv = [t[:, src].clone() for t in kv]
        from flexkv_b200.common.block import SequenceMeta
        m = cpu.match(SequenceMeta(tok, T))
        assert cpu.index.swa_lock_cnt(m.last_swa_node) == 0          # the write-through lock is gone
        # the host tier forgets everything (its snapshot slot comes back), the SSD tier keeps both
        mgr._clear_cpu_cache()
        assert cpu.swa_pool.num_used == 0 and ssd.index.total_swa_slots() == 1
        tid, mask = mgr.get_match(tok, swa_aware=True)
        assert int(mask.sum()) == 5 * T
        kinds = sorted((o.transfer_type.value, o.is_swa) for o in mgr.kv_task_engine.tasks[tid].graph.ops()
                       if o.transfer_type.value != "Virtual")
        assert kinds == [("DISK2H", False), ("DISK2H", True), ("H2D", False), ("H2D", True)]
        dst = np.arange(40, 45)
        for t in kv:
            t[:, dst] = 0
        for t in swa:
            t[11] = 0
        mgr.launch(tid, slots(dst), swa_slot_mappings=[slots([11])])
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], want_kv[l])
        for l in range(SWA_LAYERS):
            assert torch.equal(swa[l][11], want_page[l])
        assert cpu.swa_pool.num_used == 0                               # the staging slot went back
        ms = ssd.match(SequenceMeta(tok, T))
        assert ssd.index.swa_lock_cnt(ms.last_swa_node) == 0
        # a launch without window pages drops the whole chain, SSD hop included
        tok2 = tok + 1
        tid, mask = mgr.put_match(tok2)
        mgr.launch(tid, slots([20, 21, 22, 23, 24]))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert ssd.swa_pool.num_used == 1 and ssd.index.total_swa_slots() == 1
    finally:
        mgr.shutdown()


STATE_LAYERS, STATE_BYTES = 2, 32


def _state_tensors(dev, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 256, (16, STATE_BYTES), dtype=torch.uint8, generator=g).to(dev) for _ in range(STATE_LAYERS)]


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("remote_registration", [False, True])
def test_sidecar_state_travels_in_the_same_slot(device, remote_registration):
    """A sidecar group (state kept beside the window KV, other layer count and page size) is saved and restored
    with the slot; the window tensors may be registered by the engine rank over the registration channel."""
    from flexkv_b200 import KVTPClient
    from flexkv_b200.server.utils import unique_ipc_endpoint
    shape = KVShape("s", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_swa_transfer=True,
                      swa=SWAPoolConfig(enabled=True, num_slots=4, num_swa_layers=SWA_LAYERS,
                                        bytes_per_token_per_layer=PAGE_BYTES // T, evict_ratio=0.25,
                                        sidecar_groups=[(STATE_LAYERS, STATE_BYTES)],
                                        wait_for_registration=remote_registration))
    dev = "cpu" if device == "cpu" else torch.device(device)
    reg = unique_ipc_endpoint("swareg") if remote_registration else None
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True, gpu_register_port=reg)
    kv, layout = alloc_paged_cache(shape, 64, dev, "vllm", fill="normal", seed=5)
    g = torch.Generator().manual_seed(9)
    swa = [torch.randint(0, 256, (16, PAGE_BYTES), dtype=torch.uint8, generator=g).to(dev) for _ in range(SWA_LAYERS)]
    state = _state_tensors(dev, 13)
    client = None
    if remote_registration:
        mgr.start()
        client = KVTPClient(reg, dp_client_id=0, device_id=0, tp_rank=0)
        client.register_to_server(kv, layout, mode="same_process")
        client.register_swa_to_server(state, group_id=1, mode="same_process")      # any order
        client.register_swa_to_server(swa, group_id=0, mode="same_process")
    else:
        mgr.register_gpu_tensors(kv, layout)
        mgr.register_swa_tensors(swa)
        mgr.register_swa_tensors(state, group_id=1)
        mgr.start()
    mgr.wait_ready(30)
    try:
        pool = mgr.transfer_manager.storage.swa_host
        assert pool.rank_slot_bytes == SWA_LAYERS * PAGE_BYTES + STATE_LAYERS * STATE_BYTES
        assert pool.group_offsets == [0, SWA_LAYERS * PAGE_BYTES]
        tok = np.arange(4 * T, dtype=np.int64) + 300
        assert put(mgr, tok, np.array([3, 9, 1, 30]), page=5).status.value == "success"
        want_page = [t[5].clone() for t in swa]
        want_state = [t[5].clone() for t in state]
        for t in swa + state:
            t[11] = 0
            t[5] = 0
        tid, mask = mgr.get_match(tok, swa_aware=True)
        assert int(mask.sum()) == 4 * T
        mgr.launch(tid, slots(np.arange(40, 44)), swa_slot_mappings=[slots([11])])
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(SWA_LAYERS):
            assert torch.equal(swa[l][11], want_page[l])
        for l in range(STATE_LAYERS):
            assert torch.equal(state[l][11], want_state[l])
    finally:
        mgr.shutdown()


def test_sidecar_registration_must_match_the_configured_geometry():
    shape = KVShape("s", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_swa_transfer=True,
                      swa=SWAPoolConfig(enabled=True, num_slots=4, num_swa_layers=SWA_LAYERS,
                                        bytes_per_token_per_layer=PAGE_BYTES // T,
                                        sidecar_groups=[(STATE_LAYERS, STATE_BYTES)]))
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=5)
    mgr.register_gpu_tensors(kv, layout)
    mgr.register_swa_tensors([torch.zeros(16, PAGE_BYTES, dtype=torch.uint8) for _ in range(SWA_LAYERS)])
    mgr.register_swa_tensors([torch.zeros(16, STATE_BYTES * 2, dtype=torch.uint8) for _ in range(STATE_LAYERS)],
                             group_id=1)
    mgr.start()
    try:
        with pytest.raises(RuntimeError, match="window group 1"):
            mgr.wait_ready(30)
    finally:
        mgr.shutdown()


def test_remote_window_tier_serves_the_snapshot_after_the_host_copy_is_gone(tmp_path):
    """Same as the SSD window tier, one level further out: block-addressed remote files plus a window file."""
    shape = KVShape("s", 2, 2, 16, tokens_per_block=T)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_remote=True, num_remote_blocks=64,
                      remote_cache_path=str(tmp_path), remote_file_num=2, enable_swa_transfer=True,
                      swa=SWAPoolConfig(enabled=True, num_slots=4, num_remote_slots=8, num_swa_layers=SWA_LAYERS,
                                        bytes_per_token_per_layer=PAGE_BYTES // T, evict_ratio=0.25))
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=5)
    mgr.register_gpu_tensors(kv, layout)
    g = torch.Generator().manual_seed(9)
    swa = [torch.randint(0, 256, (16, PAGE_BYTES), dtype=torch.uint8, generator=g) for _ in range(SWA_LAYERS)]
    mgr.register_swa_tensors(swa)
    mgr.start(); mgr.wait_ready(30)
    try:
        gce = mgr.kv_task_engine.cache_engine
        cpu, rem = gce.cpu_cache_engine, gce.remote_cache_engine
        tok = np.arange(5 * T, dtype=np.int64) + 900
        src = np.array([3, 9, 1, 30, 12])
        tid, mask = mgr.put_match(tok)
        kinds = sorted((o.transfer_type.value, o.is_swa) for o in mgr.kv_task_engine.tasks[tid].graph.ops()
                       if o.transfer_type.value != "Virtual")
        assert kinds == [("D2H", False), ("D2H", True), ("H2REMOTE", False), ("H2REMOTE", True)]
        mgr.launch(tid, slots(src), swa_slot_mappings=[slots([5])])
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert rem.index.total_swa_slots() == 1 and rem.swa_pool.num_used == 1
        assert (tmp_path / "flexkv_remote_swa.bin").stat().st_size == 8 * SWA_LAYERS * PAGE_BYTES
        want_page = [t[5].clone() for t in swa]
        want_kv = [t[:, src].clone() for t in kv]
        mgr._clear_cpu_cache()
        assert cpu.swa_pool.num_used == 0
        tid, mask = mgr.get_match(tok, swa_aware=True)
        assert int(mask.sum()) == 5 * T
        kinds = sorted((o.transfer_type.value, o.is_swa) for o in mgr.kv_task_engine.tasks[tid].graph.ops()
                       if o.transfer_type.value != "Virtual")
        assert kinds == [("H2D", False), ("H2D", True), ("REMOTE2H", False), ("REMOTE2H", True)]
        dst = np.arange(40, 45)
        for t in kv:
            t[:, dst] = 0
        for t in swa:
            t[11] = 0
        mgr.launch(tid, slots(dst), swa_slot_mappings=[slots([11])])
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], want_kv[l])
        for l in range(SWA_LAYERS):
            assert torch.equal(swa[l][11], want_page[l])
        assert cpu.swa_pool.num_used == 0
    finally:
        mgr.shutdown()
