"""The connector driven through vLLM's OWN built-in shim class with vLLM's OWN request, scheduler-output, block and
connector-output objects (the installed vLLM, on CPU): what the engine calls is what runs here. Only the engine
configuration object is bypassed (building one needs a model checkpoint); the data plane is the host stand-in."""
import importlib.util
import time

import numpy as np
import pytest
import torch

if importlib.util.find_spec("vllm") is None:
    pytest.skip("vllm is not installed", allow_module_level=True)

from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.integration.config import FlexKVConfig  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config  # noqa: E402

T = 4


def _vllm():
    try:
        from vllm.distributed.kv_transfer.kv_connector.v1.flexkv_connector import FlexKVConnectorV1
        from vllm.sampling_params import SamplingParams
        from vllm.v1.core.kv_cache_manager import KVCacheBlocks
        from vllm.v1.core.kv_cache_utils import KVCacheBlock
        from vllm.v1.core.sched.output import SchedulerOutput
        from vllm.v1.outputs import KVConnectorOutput
        from vllm.v1.request import Request, RequestStatus
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"this vllm does not expose the pieces the test drives: {e!r}")
    return locals()


def test_offload_and_restore_through_vllms_own_classes(monkeypatch, tmp_path):
    import sys
    import os
    v = _vllm()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(os.path.join(root, "compat"))           # `import flexkv` resolves to this package
    from flexkv.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVSchedulerConnector

    shape = KVShape("v", 2, 2, 16, tokens_per_block=T)
    cfg = FlexKVConfig()
    cfg.model_config = make_model_config(shape)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=32)
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", fill="normal", seed=3)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    impl = FlexKVConnectorV1Impl.__new__(FlexKVConnectorV1Impl)
    impl.is_scheduler, impl.scheduler, impl.worker = True, FlexKVSchedulerConnector(cfg, kv_manager=mgr), None
    impl._finished_sending, impl._finished_recving, impl._previous_scheduled = set(), set(), set()
    shim = v["FlexKVConnectorV1"].__new__(v["FlexKVConnectorV1"])        # vLLM's class, our implementation behind it
    shim._flexkv_connector = impl

    def request(rid, tokens):
        return v["Request"](request_id=rid, prompt_token_ids=[int(t) for t in tokens],
                            sampling_params=v["SamplingParams"](max_tokens=1), pooling_params=None)

    def blocks(ids):
        return v["KVCacheBlocks"](blocks=([v["KVCacheBlock"](block_id=int(i)) for i in ids],))

    def step_until(name, rid):
        out = v["KVConnectorOutput"]()
        t0 = time.time()
        while rid not in (getattr(out, name) or ()) and time.time() - t0 < 10:
            shim.update_connector_output(out)
            time.sleep(0.002)
        return out

    try:
        tok = np.arange(300, 300 + 6 * T + 1)
        r1 = request("a", tok)
        assert shim.get_num_new_matched_tokens(r1, 0) == (0, False)
        r1.status = v["RequestStatus"].FINISHED_LENGTH_CAPPED
        keep, params = shim.request_finished(r1, [10, 11, 12, 13, 14, 15, 16])
        assert keep is True and params is None
        meta = shim.build_connector_meta(v["SchedulerOutput"].make_empty())
        from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorMetadata
        assert isinstance(meta, KVConnectorMetadata)
        out = step_until("finished_sending", "a")
        assert "a" in out.finished_sending
        # the same prompt again: 2 blocks computed by the engine, 4 restored
        r2 = request("b", tok)
        n, is_async = shim.get_num_new_matched_tokens(r2, 2 * T)
        assert (n, is_async) == (4 * T, True)
        saved = [t.clone() for t in kv]
        shim.update_state_after_alloc(r2, blocks([40, 41, 42, 43, 44, 45, 46]), n)
        shim.build_connector_meta(v["SchedulerOutput"].make_empty())
        out = step_until("finished_recving", "b")
        assert "b" in out.finished_recving
        for l in range(2):
            assert torch.equal(kv[l][:, [42, 43, 44, 45]], saved[l][:, [12, 13, 14, 15]])
        assert shim.get_block_ids_with_load_errors() == set()
        from vllm.distributed.kv_transfer.kv_connector.v1.metrics import KVConnectorStats
        stats = shim.get_kv_connector_stats()
        assert isinstance(stats, KVConnectorStats) and not stats.is_empty()
        assert stats.data["num_get_requests"] == 2 and stats.data["num_put_requests"] == 1
        assert stats.data["num_flexkv_matched_tokens"] == 4 * T
        again = shim.get_kv_connector_stats()                # an interval in which nothing happened
        assert again.is_empty() and again.data["num_get_requests"] == 0
        total = stats.aggregate(again).reduce()              # what the engine's logger does with the records
        assert total["num_get_requests"] == 2
        assert abs(total["get_flexkv_match_ratio"] - 4 * T / total["num_get_query_tokens"]) < 1e-9
        import pickle
        assert pickle.loads(pickle.dumps(stats)).data == stats.data
        # the worker side counts nothing but must not look empty to the engine
        impl.is_scheduler = False
        sentinel = shim.get_kv_connector_stats()
        impl.is_scheduler = True
        assert isinstance(sentinel, KVConnectorStats) and sentinel.is_empty() and sentinel.aggregate(stats) is stats
        assert not v["KVConnectorOutput"](kv_connector_stats=sentinel).is_empty()
        assert list(shim.take_events()) == []                    # events are off unless asked for
        impl.scheduler.enable_kv_events()
        r4 = request("d", np.arange(7000, 7000 + 3 * T + 1))
        r4.status = v["RequestStatus"].FINISHED_STOPPED
        assert shim.request_finished(r4, [20, 21, 22, 23])[0] is True
        shim.build_connector_meta(v["SchedulerOutput"].make_empty())
        step_until("finished_sending", "d")
        from vllm.distributed.kv_events import BlockStored, KVCacheEvent, KVEventBatch
        events = list(shim.take_events())
        assert events and all(isinstance(e, KVCacheEvent) for e in events)
        stored = [e for e in events if isinstance(e, BlockStored)]
        assert sum(len(e.block_hashes) for e in stored) == 3 and stored[0].block_size == T and stored[0].medium == "CPU"
        import msgspec
        msgspec.msgpack.encode(KVEventBatch(ts=0.0, events=events))     # what the engine's publisher does with them
        # an aborted request leaves nothing behind
        r3 = request("c", np.arange(9000, 9000 + 5 * T))
        r3.status = v["RequestStatus"].FINISHED_ABORTED
        assert shim.request_finished(r3, [1, 2, 3, 4, 5]) == (False, None)
    finally:
        shim.shutdown()


def test_connector_is_built_from_vllms_own_config_objects(monkeypatch, tmp_path):
    """vLLM's real ModelConfig / ParallelConfig / CacheConfig / KVTransferConfig (a six-layer Llama described by a
    local config.json, no weights) feed the scheduler-side connector: geometry and tier sizes come out right.
    (A whole VllmConfig cannot be built without a device; its parts can.)"""
    import json
    import os
    from types import SimpleNamespace as NS
    try:
        from vllm.config import CacheConfig as VCache, KVTransferConfig, ModelConfig as VModel, ParallelConfig
        from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vllm config classes not importable: {e!r}")
    model_dir = tmp_path / "tiny"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 256, "intermediate_size": 512,
        "num_attention_heads": 8, "num_key_value_heads": 4, "num_hidden_layers": 6, "vocab_size": 1000,
        "max_position_embeddings": 2048, "rms_norm_eps": 1e-5, "torch_dtype": "bfloat16", "head_dim": 32}))
    try:
        mc = VModel(model=str(model_dir), tokenizer=str(model_dir), skip_tokenizer_init=True, dtype="bfloat16")
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"this vllm cannot build a ModelConfig on a box without a device: {e!r}")
    vc = NS(model_config=mc, parallel_config=ParallelConfig(), cache_config=VCache(block_size=16),
            kv_transfer_config=KVTransferConfig(kv_connector="FlexKVConnectorV1", kv_role="kv_both"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(os.path.join(root, "compat"))
    monkeypatch.delenv("FLEXKV_CONFIG_PATH", raising=False)
    monkeypatch.setenv("FLEXKV_CPU_CACHE_GB", "0.01")                      # fractional sizes are accepted
    monkeypatch.setenv("FLEXKV_SERVER_RECV_PORT", f"ipc://{tmp_path}/srv")
    from flexkv.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl
    impl = FlexKVConnectorV1Impl(vc, KVConnectorRole.SCHEDULER)
    try:
        m, c = impl.scheduler.cfg.model_config, impl.scheduler.cfg.cache_config
        assert (m.num_layers, m.num_kv_heads, m.head_size, m.tp_size, m.use_mla) == (6, 4, 32, 1, False)
        assert m.dtype == torch.bfloat16 and c.tokens_per_block == 16
        block_bytes = 6 * 2 * 16 * 4 * 32 * 2
        assert c.num_cpu_blocks == int(0.01 * (1 << 30)) // block_bytes
    finally:
        impl.shutdown()


def test_mla_geometry_is_read_off_vllms_own_model_config(tmp_path):
    """A DeepSeek-V3-shaped config through vLLM's real ModelConfig: one latent head of kv_lora_rank + rope width,
    no K/V axis, whatever the tensor-parallel size."""
    import json
    from types import SimpleNamespace as NS
    try:
        from vllm.config import CacheConfig as VCache, ModelConfig as VModel, ParallelConfig
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vllm config classes not importable: {e!r}")
    d = tmp_path / "ds"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({
        "architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3", "hidden_size": 256,
        "intermediate_size": 512, "moe_intermediate_size": 128, "num_attention_heads": 8, "num_key_value_heads": 8,
        "num_hidden_layers": 4, "vocab_size": 1000, "kv_lora_rank": 512, "q_lora_rank": 128, "qk_rope_head_dim": 64,
        "qk_nope_head_dim": 128, "v_head_dim": 128, "n_routed_experts": 4, "n_shared_experts": 1,
        "num_experts_per_tok": 2, "first_k_dense_replace": 1, "max_position_embeddings": 2048, "rms_norm_eps": 1e-6,
        "torch_dtype": "bfloat16"}))
    try:
        mc = VModel(model=str(d), tokenizer=str(d), skip_tokenizer_init=True, dtype="bfloat16")
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"this vllm cannot build the model config here: {e!r}")
    assert mc.use_mla
    cfg = FlexKVConfig()
    cfg.post_init_from_vllm_config(NS(model_config=mc, parallel_config=ParallelConfig(tensor_parallel_size=2),
                                      cache_config=VCache(block_size=64)))
    m = cfg.model_config
    assert (m.num_layers, m.num_kv_heads, m.head_size, m.kv_dim, m.tp_size, m.use_mla) == (4, 1, 576, 1, 2, True)
    assert cfg.cache_config.tokens_per_block == 64
