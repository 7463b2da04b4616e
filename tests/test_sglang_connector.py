"""SGLang connector on CPU: single rank end to end, the layer-done counter, and
the store protocol across two gloo ranks (reference: tests/test_sglang_connector.py,
test_sglang_store_protocol.py, run_sglang_store_protocol_distributed.py)."""
import os
import struct
import subprocess
import sys
import threading

import numpy as np
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.integration.config import FlexKVConfig
from flexkv_b200.integration.sglang.comm import FlexKVLayerDoneCounter
from flexkv_b200.integration.sglang.connector import FlexKVConnector
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T = 4


def test_single_rank_store_lookup_retrieve():
    shape = KVShape("sg", 2, 2, 16, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "sglang", fill="normal", seed=90)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    conn = FlexKVConnector(cfg, page_size=T, kv_manager=mgr, register=False)
    try:
        tok = list(range(300, 300 + 5 * T + 3))
        pages = np.array([9, 2, 33, 4, 17])
        slot = np.concatenate([np.repeat(pages, T) * T + np.tile(np.arange(T), 5), [0, 1, 2]])
        assert conn.store_kv("r1", tok, slot) == 5 * T
        assert conn.wait_store("r1") and conn.check_completed_stores() == []
        saved = [t.clone() for t in kv]
        for t in kv:
            t.zero_()
        assert conn.lookup_kv("r2", tok, num_computed_tokens=T) == 4 * T
        dst = np.array([40, 41, 42, 43])
        assert conn.retrieve_kv("r2", np.repeat(dst, T) * T + np.tile(np.arange(T), 4)) == 4 * T
        for i in range(4):          # K buffers then V buffers
            assert torch.equal(kv[i][dst], saved[i][pages[1:]])
        assert conn.lookup_kv("r3", list(range(9000, 9016))) == 0
        conn.reset()
        assert conn.lookup_kv("r4", tok) == 0
    finally:
        conn.shutdown()


def test_layer_done_counter_counts_one_unit_per_restore_per_layer():
    c = FlexKVLayerDoneCounter(num_layers=3, num_counters=3)
    try:
        p = c.update_producer()
        c.register_task(11, p)
        c.register_task(12, p)                         # two restores feed the same forward pass
        c.set_consumer(11)
        fds = c.fds_per_counter()[p]

        def worker():
            for l in range(3):
                for _ in range(2):
                    os.write(fds[l], struct.pack("Q", 1))

        th = threading.Thread(target=worker)
        th.start()
        for l in range(3):
            c.wait_until(l, timeout=5)                 # returns only after both units of the layer arrived
        th.join()
        q = c.update_producer()
        assert q != p
        c.register_task(13, q)
        c.rollback_prepared_transfer(13)
        assert c.events[q].pending_transfers() == 0
    finally:
        c.close()


WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.integration.config import FlexKVConfig
from flexkv_b200.integration.sglang.connector import FlexKVConnector
from flexkv_b200.integration.sglang.comm import FlexKVComm
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
dist.init_process_group("gloo")
rank = dist.get_rank()
T = 4
shape = KVShape("sg", 2, 2, 16, tokens_per_block=T)
cfg = FlexKVConfig()
cfg.model_config = make_model_config(shape)
cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
mgr = None
if rank == 0:
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "sglang", fill="normal", seed=1)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
conn = FlexKVConnector(cfg, page_size=T, comm=FlexKVComm(tp_size=2), kv_manager=mgr, register=False)
tok = list(range(5 * T))
slot = np.repeat(np.arange(5), T) * T + np.tile(np.arange(T), 5)
moved = conn.store_kv("a", tok, slot)            # decided on the leader, identical on both ranks
ok = conn.wait_store("a")
hit = conn.lookup_kv("b", tok, num_computed_tokens=T)
got = conn.retrieve_kv("b", slot[T:] + 100)
assert (moved, ok, hit, got) == (5 * T, True, 4 * T, 4 * T), (rank, moved, ok, hit, got)
assert conn.comm.all_reduce_min(10 + rank) == 10
conn.reset()
conn.shutdown()
dist.barrier()
dist.destroy_process_group()
sys.stdout.write("rank%d-ok\n" % rank); sys.stdout.flush()
"""


def test_store_protocol_across_two_gloo_ranks(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER.replace("%(root)r", repr(ROOT)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29621", str(script)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, PYTHONPATH=ROOT))
    assert p.returncode == 0, p.stdout[-1500:] + p.stderr[-1500:]
    assert "rank0-ok" in p.stdout and "rank1-ok" in p.stdout


PP_WORKER = r'''
import sys
sys.path.insert(0, "ROOT")
import torch.distributed as dist
from flexkv_b200.integration.sglang.comm import FlexKVComm
dist.init_process_group("gloo")
c = FlexKVComm(tp_size=2, pp_size=2)
got = c.scatter_pp({"plan": 42} if c.rank == 0 else None)
assert got == ({"plan": 42} if c.rank in (0, 2) else None), (c.rank, got)
assert c.all_reduce_min(10 + c.rank) == 10
sys.stdout.write("PP_OK %d\n" % c.rank)
dist.destroy_process_group()
'''


def test_pipeline_stage_leaders_receive_the_plan(tmp_path):
    script = tmp_path / "pp_worker.py"
    script.write_text(PP_WORKER.replace("ROOT", ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", "29567", str(script)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, PYTHONPATH=ROOT))
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("PP_OK") == 4


def test_layer_done_counter_guards_rank_skewed_batches():
    """A follower registers on the set the leader chose; a set that a forward pass already consumes, or a task
    registered twice, is refused; an empty selection goes back to the ring
    (reference: flexkv/integration/sglang/comm.py:798-925)."""
    import pytest
    c = FlexKVLayerDoneCounter(num_layers=2, num_counters=3)
    try:
        assert c.expected_transfer_count(1) == 0
        c.register_task_with_explicit_counter_id(5, 1)             # the leader said: set 1
        assert c.expected_transfer_count(1) == 1
        with pytest.raises(RuntimeError):
            c.register_task_with_explicit_counter_id(5, 1)
        with pytest.raises(ValueError):
            c.expected_transfer_count(7)
        c.set_consumer(5)
        fds = c.fds_per_counter()[1]
        for l in range(2):
            os.write(fds[l], struct.pack("Q", 1))
        c.wait_until(0, timeout=5)
        with pytest.raises(RuntimeError):                          # the forward pass is already reading set 1
            c.register_task_with_explicit_counter_id(6, 1)
        c.wait_until(1, timeout=5)
        assert c.events[1].finished and c.expected_transfer_count(1) == 0      # back in the ring
        p = c.update_producer()
        c.abort_unregistered_selection(p)                          # the leader's plan turned out empty
        assert c.events[p].finished and c.update_producer() == p
        c.register_task(9, p)
        with pytest.raises(RuntimeError):
            c.abort_unregistered_selection(p)
    finally:
        c.close()


def test_the_reference_integrations_calling_convention_drives_the_same_connector():
    """The calls of the reference's SGLang patch, argument for argument (flexkv/integration/sglang/
    sglang_flexkv_connector.patch: lookup with a token mask and keyword request ids, store that returns the id of
    the store in flight or -1, the argument-less sweep of launched loads, prefetch with the engine's request id)."""
    shape = KVShape("sg", 2, 2, 16, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "sglang", fill="normal", seed=91)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    conn = FlexKVConnector(cfg, page_size=T, kv_manager=mgr, register=False)
    try:
        assert conn.enable_layerwise is False
        tok = list(range(700, 700 + 5 * T))
        pages = np.array([9, 2, 33, 4, 17])
        indices = torch.from_numpy(np.repeat(pages, T) * T + np.tile(np.arange(T), 5))
        task_id = conn.store_kv("r1:flexkv-store:0", tok, indices, sglang_req_id="r1")
        assert isinstance(task_id, int) and task_id >= 0
        import time
        t0 = time.time()
        done = []
        while not done and time.time() - t0 < 10:
            done = conn.check_completed_stores()
            time.sleep(0.002)
        assert done == ["r1:flexkv-store:0"]
        assert conn.store_kv("r1:flexkv-store:1", tok, indices, sglang_req_id="r1") == -1     # nothing new to store
        saved = [t.clone() for t in kv]
        for t in kv:
            t.zero_()
        token_mask = torch.zeros(len(tok), dtype=torch.bool)
        token_mask[T:] = True                                        # the first page is on the GPU already
        tid, hit = conn.lookup_kv(tok, token_mask, rid="r2", sglang_req_id="r2")
        assert tid >= 0 and hit == 4 * T
        dst = np.array([40, 41, 42, 43])
        assert conn.retrieve_kv("r2", torch.from_numpy(np.repeat(dst, T) * T + np.tile(np.arange(T), 4))) == 4 * T
        for i in range(4):
            assert torch.equal(kv[i][dst], saved[i][pages[1:]])
        # a lookup nobody tracks holds nothing afterwards
        tid, hit = conn.lookup_kv(tok, token_mask)
        assert hit == 4 * T and not conn._pending_loads
        # a miss, a released hit, the sweep and the prefetch form
        assert conn.lookup_kv(list(range(9000, 9016)), torch.ones(16, dtype=torch.bool), rid="r3")[1] == 0
        conn.lookup_kv(tok, token_mask, rid="r4", sglang_req_id="r4")
        conn.release_pending("r4")
        assert not conn._pending_loads
        assert conn.drain_launched_loads() is None
        conn.prefetch_async("r5", tok, sglang_req_id="r5")
        conn.cancel_prefetch("r5")
    finally:
        conn.shutdown()


def test_the_reference_constructor_reads_the_engines_objects():
    """``FlexKVConnector(sgl_model_config=, server_args=, page_size=, kvcache=, tp_rank=, ..., attn_tp_group=, ...)``
    as the reference's SGLang patch builds it: geometry from the engine's model config, group sizes from the
    engine's groups, dtype from the server arguments."""
    from types import SimpleNamespace as NS
    model = NS(num_hidden_layers=2, num_key_value_heads=4, head_dim=16, dtype=torch.bfloat16)
    args = NS(kv_cache_dtype="auto", dp_size=1)
    group = NS(world_size=2)                                      # the engine's group coordinator
    shape = KVShape("sg", 2, 2, 16, tokens_per_block=T)           # 4 KV heads over 2 TP ranks
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "sglang", fill="zeros")
    probe = FlexKVConfig()
    probe.post_init_from_sglang_config(args, model, T, tp_size=2)
    mgr = KVManager(probe.model_config, CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    mgr.register_gpu_tensors(kv, layout, tp_rank=0)
    kv1, _ = alloc_paged_cache(shape, 64, "cpu", "sglang", fill="zeros")
    mgr.register_gpu_tensors(kv1, layout, tp_rank=1)
    mgr.start(); mgr.wait_ready(30)
    conn = FlexKVConnector(sgl_model_config=model, server_args=args, page_size=T, kvcache=None, tp_rank=0, dp_rank=0,
                           pp_rank=0, attn_cp_rank=0, pp_group=None, attn_tp_group=group, attn_cp_group=None,
                           kv_manager=mgr, register=False)
    try:
        m = conn.cfg.model_config
        assert (m.num_layers, m.num_kv_heads, m.head_size, m.tp_size, m.cp_size, m.pp_size) == (2, 4, 16, 2, 1, 1)
        assert conn.T == T and conn.tp_size == 2 and conn.enable_layerwise is False
        assert conn.lookup_kv(list(range(16)), torch.ones(16, dtype=torch.bool), rid="x") == (-1, 0)
    finally:
        conn.shutdown()
    import pytest
    with pytest.raises(TypeError):
        FlexKVConnector(page_size=T)
