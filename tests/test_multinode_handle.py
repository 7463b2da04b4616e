"""A tensor-parallel group split over two nodes: the master plans, both nodes move their
own rank's slice, a graph is finished only when both reported
(reference: flexkv/transfer_manager.py:529-908,1279-1468)."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4
HERE = os.path.dirname(os.path.abspath(__file__))


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def test_two_node_tp_group_round_trip(tmp_path):
    pytest.importorskip("zmq")
    cmd, res, qry = (f"ipc://{tmp_path}/{n}.sock" for n in ("cmd", "res", "qry"))
    out = str(tmp_path / "remote.pt")
    child = subprocess.Popen([sys.executable, os.path.join(HERE, "mp_workers", "remote_tm_worker.py"), cmd, res, qry,
                              out], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    mgr = None
    try:
        shape = KVShape("mn", 2, 4, 16, tokens_per_block=T)
        mgr = KVManager(make_model_config(shape, tp_size=2, nnodes=2), CacheConfig(tokens_per_block=T, num_cpu_blocks=24),
                        require_gpu=True, remote_transfer_endpoints=[(cmd, res, qry)])
        kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", tp_size=2, fill="normal", seed=5)
        mgr.register_gpu_tensors(kv, layout, tp_rank=0)
        mgr.start()
        mgr.wait_ready(60)
        tok = np.arange(5 * T, dtype=np.int64)
        src = np.array([3, 9, 1, 30, 12])
        dst = np.arange(40, 45)
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True, timeout=30)[tid].status.value == "success"
        for t in kv:
            t[:, dst] = 0
        tid = mgr.get_async(tok, slots(dst))
        assert mgr.wait(tid, timeout=30)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], kv[l][:, src])
    finally:
        if mgr is not None:
            mgr.shutdown()
        try:
            text, _ = child.communicate(timeout=30)
        except subprocess.TimeoutExpired:
            child.kill()
            text, _ = child.communicate()
    assert child.returncode == 0, text[-2000:]
    r = torch.load(out)
    for l in range(2):
        # the other node restored its own rank's slice into the same destination blocks
        assert torch.equal(r["after"][l][:, dst], r["before"][l][:, src])
        assert not torch.equal(r["before"][l][:, dst], r["before"][l][:, src])


def test_remote_node_binds_its_own_pages_from_its_ranks(tmp_path):
    """The other node numbers its GPU pages itself: graphs reach it with the GPU side unbound and run once one of
    its ranks has sent the task's page list (in either order), so the two nodes use different pages for the
    same task (flexkv/server/client.py:308-334, flexkv/kvtask.py:438-444)."""
    pytest.importorskip("zmq")
    from flexkv_b200.server.client import KVTPClient
    cmd, res, qry, reg = (f"ipc://{tmp_path}/{n}.sock" for n in ("cmd", "res", "qry", "reg"))
    out = str(tmp_path / "remote.pt")
    child = subprocess.Popen([sys.executable, os.path.join(HERE, "mp_workers", "remote_tm_worker.py"), cmd, res, qry,
                              out, reg], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    mgr = None
    rank_on_other_node = KVTPClient(reg, 0, -1, tp_rank=1)
    try:
        shape = KVShape("mn", 2, 4, 16, tokens_per_block=T)
        mgr = KVManager(make_model_config(shape, tp_size=2, nnodes=2), CacheConfig(tokens_per_block=T, num_cpu_blocks=24),
                        require_gpu=True, remote_transfer_endpoints=[(cmd, res, qry, True)])
        kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", tp_size=2, fill="normal", seed=5)
        mgr.register_gpu_tensors(kv, layout, tp_rank=0)
        mgr.start()
        mgr.wait_ready(60)
        tok = np.arange(5 * T, dtype=np.int64)
        src, dst = np.array([3, 9, 1, 30, 12]), np.arange(40, 45)
        r_src, r_dst = np.array([50, 2, 17, 8, 61]), np.arange(20, 25)          # the other node's own pages
        tid = mgr.put_async(tok, slots(src))
        time.sleep(0.3)                                   # the graph is already waiting over there
        rank_on_other_node.set_slot_mapping(tid, slots(r_src))
        assert mgr.wait(tid, completely=True, timeout=30)[tid].status.value == "success"
        tid, mask = mgr.get_match(tok)
        rank_on_other_node.set_slot_mapping(tid, slots(r_dst))      # this time the page list arrives first
        time.sleep(0.3)
        mgr.launch(tid, slots(dst))
        assert mgr.wait(tid, timeout=30)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv[l][:, dst], kv[l][:, src])
    finally:
        if mgr is not None:
            mgr.shutdown()
        rank_on_other_node.shutdown()
        try:
            text, _ = child.communicate(timeout=30)
        except subprocess.TimeoutExpired:
            child.kill()
            text, _ = child.communicate()
    assert child.returncode == 0, text[-2000:]
    r = torch.load(out)
    for l in range(2):
        assert torch.equal(r["after"][l][:, r_dst], r["before"][l][:, r_src])
        assert torch.equal(r["after"][l][:, dst], r["before"][l][:, dst])       # the master's pages were not used there
