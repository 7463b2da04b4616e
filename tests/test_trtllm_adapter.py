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


def test_namespace_rule_and_request_wrapper():
    from flexkv_b200.integration.tensorrt_llm.utils import RequestWrapper, extract_namespace, physical_device_id
    r = NS(request_id=5, lora_task_id=123, cache_salt_id="session_1", namespace_info="tenant_A| user_1 |",
           get_tokens=lambda: [[1, 2, 3, 4, 5]], prompt_len=4, num_connector_matched_tokens=2,
           is_finished=True, is_finished_normal=lambda: False)
    assert extract_namespace(r) == ["123", "session_1", "tenant_A", "user_1"]
    assert extract_namespace(NS()) is None and extract_namespace(NS(namespace_info=7)) == ["7"]
    w = RequestWrapper(r)
    assert w.req_id == 5 and w.all_token_ids == [1, 2, 3, 4, 5] and w.num_prompt_tokens == 4
    assert w.np_token_ids.dtype == np.int64 and w.np_token_ids is w.np_token_ids       # converted once
    assert w.num_new_matched_tokens == 2 and w.is_finished() and not w.is_finished_normal()
    assert w.namespace_info == ["123", "session_1", "tenant_A", "user_1"]
    with pytest.raises(ValueError):
        RequestWrapper(NS(get_tokens=lambda: [[1], [2]])).all_token_ids            # beam search
    assert physical_device_id(1, "4,6") == 6 and physical_device_id(3, "4,6") == 3 and physical_device_id(2, None) == 2
    assert physical_device_id(0, "GPU-abc") == 0


def test_namespaces_isolate_requests_with_the_same_tokens():
    conn, pool, mgr = make()
    try:
        tok = np.arange(900, 900 + 4 * T)
        a = NS(py_request_id=21, request_id=None, get_tokens=lambda beam: list(tok), lora_task_id=1,
               namespace_info="tenant_A")
        assert conn.request_finished(a, [1, 2, 3, 4]) is True
        assert "21" in drain(conn, "finished_sending", 21)
        same = NS(py_request_id=22, request_id=None, get_tokens=lambda beam: list(tok), lora_task_id=1,
                  namespace_info="tenant_A")
        other = NS(py_request_id=23, request_id=None, get_tokens=lambda beam: list(tok), lora_task_id=1,
                   namespace_info="tenant_B")
        assert conn.get_num_new_matched_tokens(other, 0)[0] == 0           # another tenant sees nothing
        n, _ = conn.get_num_new_matched_tokens(same, 0)
        assert n > 0 and conn.tasks["22"].num_new_matched_tokens == n and conn.tasks["22"].match_cost >= 0
        meta = conn.build_connector_meta()
        assert isinstance(meta.finished_sending, list) and meta["finished_recving"] == set(meta.finished_recving)
    finally:
        conn.shutdown()
        mgr.shutdown()


def test_worker_connector_reports_the_bound_metadata(tmp_path):
    from flexkv_b200.integration.tensorrt_llm.meta import FlexKVConnectorMetadata
    from flexkv_b200.integration.tensorrt_llm.trtllm_adapter import FlexKVWorkerConnector
    shape = KVShape("t", L, H, D, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=8)
    cfg.gpu_register_port = f"ipc://{tmp_path}/reg"
    w = FlexKVWorkerConnector(flexkv_config=cfg)
    try:
        assert w.remote_process is None and w.get_finished() == ([], [])
        w.bind_connector_meta(FlexKVConnectorMetadata(["3"], ["4", "5"]))
        assert w.get_finished([9], [9]) == (["3"], ["4", "5"])
        with pytest.raises(ValueError):
            w.register_kv_caches(torch.zeros(4, L, 2, 7))
    finally:
        w.shutdown()


def test_a_manager_configured_from_tensorrt_llm_keeps_the_data_plane_out_of_the_serving_process(monkeypatch):
    """TensorRT-LLM owns MPI in its processes, so a configuration read from it asks for the data plane in a child
    process; an explicit FLEXKV_TRANSFER_MANAGER_MODE or constructor argument still decides
    (reference: flexkv/integration/config.py:752, flexkv/kvtask.py:172-199)."""
    from types import SimpleNamespace as NS
    from flexkv_b200 import KVManager
    from flexkv_b200.integration.config import FlexKVConfig
    import flexkv_b200.transfer_process as tp
    made = []

    class FakeHandle:
        def __init__(self, *a, **k):
            made.append("process")

        def shutdown(self):
            pass

        def set_metrics_collector(self, c):
            pass

    monkeypatch.setattr(tp, "TransferManagerProcessHandle", FakeHandle)
    monkeypatch.delenv("FLEXKV_TRANSFER_MANAGER_MODE", raising=False)
    cfg = FlexKVConfig()
    llm = NS(model_config=NS(num_hidden_layers=2, num_key_value_heads=2, num_attention_heads=2, head_dim=16,
                             hidden_size=32, torch_dtype="bfloat16"),
             kv_cache_config=NS(dtype="auto", tokens_per_block=T))
    cfg.post_init_from_trt_config(llm, NS(tp_size=1, pp_size=1))
    assert cfg.model_config.use_trtllm_subprocess
    m = KVManager(cfg.model_config, cfg.cache_config, require_gpu=False)
    assert made == ["process"]
    m._shut = True
    m2 = KVManager(cfg.model_config, cfg.cache_config, require_gpu=False, transfer_manager_mode="thread")
    assert made == ["process"]                       # the explicit choice wins
    m2.shutdown()
