"""TensorRT-LLM connector on the single block-first pool, with stand-in request objects and the
CPU data plane (reference: flexkv/integration/tensorrt_llm/trtllm_adapter.py:29-650)."""
import time
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.integration.config import FlexKVConfig
from flexkv_b200.integration.tensorrt_llm.trtllm_adapter import FlexKVSchedulerConnector, trtllm_gpu_layout
from flexkv_b200.models import KVShape, make_model_config

T, L, H, D = 4, 3, 2, 16


def make():
    shape = KVShape("t", L, H, D, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    g = torch.Generator().manual_seed(3)
    pool = torch.randn(48, L, 2, T * H * D, generator=g).to(torch.bfloat16)      # TRT-LLM: ONE tensor
    layout = trtllm_gpu_layout(pool, L, 2, T, H, D)
    mgr.register_gpu_tensors([pool], layout)
    mgr.start(); mgr.wait_ready(30)
    return FlexKVSchedulerConnector(flexkv_config=cfg, kv_manager=mgr), pool, mgr


def llm_request(rid, tokens):
    return NS(py_request_id=rid, request_id=None, get_tokens=lambda beam: list(tokens), lora_task_id=None)


def drain(conn, key, rid, timeout=10):
    t0 = time.time()
    seen = set()
    while str(rid) not in seen and time.time() - t0 < timeout:
        seen |= conn.build_connector_meta()[key]
        time.sleep(0.005)
    return seen


def test_layout_check_rejects_a_pool_of_the_wrong_geometry():
    with pytest.raises(ValueError):
        trtllm_gpu_layout(torch.zeros(4, L, 2, 7), L, 2, T, H, D)


def test_offload_and_restore_through_the_single_pool():
    conn, pool, mgr = make()
    try:
        assert conn.is_ready()
        tok = np.arange(50, 50 + 5 * T + 1)
        r1 = llm_request(7, tok)
        assert conn.get_num_new_matched_tokens(r1, 0) == (0, False)
        assert conn.request_finished(r1, [3, 4, 5, 6, 7, 8]) is True
        assert "7" in drain(conn, "finished_sending", 7)
        r2 = llm_request(8, tok)
        n, is_async = conn.get_num_new_matched_tokens(r2, T)
        assert (n, is_async) == (4 * T, True)
        saved = pool.clone()
        conn.update_state_after_alloc(r2, [20, 21, 22, 23, 24, 25])
        assert "8" in drain(conn, "finished_recving", 8)
        assert torch.equal(pool[[21, 22, 23, 24]], saved[[4, 5, 6, 7]])
        assert torch.equal(pool[20], saved[20])                       # the block the engine computed is untouched
    finally:
        conn.shutdown()


def test_a_request_that_did_not_finish_normally_is_not_offloaded():
    conn, pool, mgr = make()
    try:
        r = llm_request(21, np.arange(900, 900 + 3 * T + 1))
        r.is_finished = True
        r.is_finished_normal = False
        assert conn.request_finished(r, [1, 2, 3, 4]) is False
        assert conn.core.stats.num_put_requests == 0
        r.is_finished_normal = True
        assert conn.request_finished(r, [1, 2, 3, 4]) is True
    finally:
        conn.shutdown()
