"""Configuration: environment table, user config files, GB -> block conversion, model geometry
(reference tests: test_config_hugepage.py, test_recompute_block_counts.py; code
flexkv/common/config.py:748-841,843-944,946-1246)."""
import json
import os

import pytest
import torch

from flexkv_b200.common import config as cfgmod
from flexkv_b200.common.config import (CacheConfig, ModelConfig, UserConfig, apply_overrides, convert_to_block_num,
                                       load_env_config, load_user_config_from_file, parse_path_list,
                                       recompute_block_counts, update_default_config_from_user_config)


def _llama():
    return ModelConfig(num_layers=32, num_kv_heads=8, head_size=128, dtype=torch.bfloat16)


def test_block_geometry_and_gb_conversion():
    m = _llama()
    assert m.token_size_in_bytes == 32 * 2 * 8 * 128 * 2            # 128 KiB per token
    assert m.block_size_in_bytes(16) == 2 << 20
    assert convert_to_block_num(1.0, 2 << 20) == 512
    mla = ModelConfig(num_layers=61, num_kv_heads=1, head_size=576, use_mla=True, dtype=torch.bfloat16)
    assert mla.block_size_in_bytes(64) == 61 * 64 * 576 * 2


def test_user_config_fills_tiers_and_rounds_ssd_blocks_to_directories(tmp_path):
    m, c = _llama(), CacheConfig(tokens_per_block=16)
    u = UserConfig(cpu_cache_gb=2, ssd_cache_gb=9, ssd_cache_dir=f"{tmp_path}/a;{tmp_path}/b;{tmp_path}/c",
                   enable_gds=True, enable_p2p_gpu=True)
    update_default_config_from_user_config(m, c, u)
    assert c.num_cpu_blocks == 1024 and c.enable_ssd and c.enable_gds and c.enable_p2p_gpu
    assert c.ssd_cache_dir == [f"{tmp_path}/a", f"{tmp_path}/b", f"{tmp_path}/c"]
    assert c.num_ssd_blocks == 4608 - 4608 % 3 and c.num_ssd_blocks % 3 == 0
    # a later change of the KV geometry re-derives the counts from the remembered sizes
    m2 = ModelConfig(num_layers=64, num_kv_heads=8, head_size=128, dtype=torch.bfloat16)
    recompute_block_counts(m2, c)
    assert c.num_cpu_blocks == 512


def test_user_config_validation():
    with pytest.raises(ValueError):
        UserConfig(cpu_cache_gb=0)
    with pytest.raises(ValueError):
        UserConfig(cpu_cache_gb=8, ssd_cache_gb=4)
    with pytest.raises(ValueError):
        CacheConfig(tokens_per_block=12)
    with pytest.raises(ValueError):
        CacheConfig(enable_gds=True, enable_ssd=False)


def test_files_json_yaml_and_overrides(tmp_path):
    pj = tmp_path / "c.json"
    pj.write_text(json.dumps({"cpu_cache_gb": 3, "override_evict_ratio": 0.25, "eviction_policy": "lfu"}))
    u = load_user_config_from_file(str(pj))
    assert u.cpu_cache_gb == 3 and u.overrides == {"override_evict_ratio": 0.25, "eviction_policy": "lfu"}
    env = load_env_config()
    apply_overrides(u, env)
    assert env.evict_ratio == 0.25 and env.eviction_policy == "lfu"
    py = tmp_path / "c.yml"
    py.write_text("cpu_cache_gb: 5\nenable_p2p_cpu: true\nno_such_key: 1\n")
    u = load_user_config_from_file(str(py))
    assert u.cpu_cache_gb == 5 and u.enable_p2p_cpu
    with pytest.raises(ValueError):
        apply_overrides(u, load_env_config())
    assert parse_path_list("/a; /b ;") == ["/a", "/b"] and parse_path_list(["/x"]) == ["/x"]


def test_environment_table(monkeypatch):
    monkeypatch.setenv("FLEXKV_TRANSFER_NUM_CTA_H2D", "12")
    monkeypatch.setenv("FLEXKV_INDEX_ACCEL", "0")
    monkeypatch.setenv("FLEXKV_LEASE_TTL_MS", "1234")
    monkeypatch.setenv("FLEXKV_TRANSFER_ENGINE", "AUTO")
    monkeypatch.setenv("FLEXKV_USE_CE_TRANSFER_H2D", "1")
    env = load_env_config()
    assert env.transfer_num_cta_h2d == 12 and env.index_accel is False and env.lease_ttl_ms == 1234
    assert env.transfer_engine == "auto" and env.use_ce_transfer_h2d is True
    from flexkv_b200.transfer.workers import _launch_cfg
    assert _launch_cfg(env, True)["engine"] == 3
    env.transfer_engine = "tma"
    assert _launch_cfg(env, True)["engine"] == 3 and _launch_cfg(env, False)["engine"] == 0


def test_model_config_parallel_layout():
    m = ModelConfig(num_layers=80, num_kv_heads=8, head_size=128, tp_size=8, pp_size=2, dp_size=2, nnodes=4)
    assert m.total_gpus == 32 and m.gpus_per_node == 8 and m.num_layers_per_pp_stage == 40
    assert m.effective_tp_size == 8 and m.effective_tp_size_per_node == 8
    two = ModelConfig(num_layers=8, num_kv_heads=8, head_size=64, tp_size=16, nnodes=2)
    assert two.nnodes_per_tp_group == 2 and two.effective_tp_size_per_node == 8
    with pytest.raises(ValueError):
        ModelConfig(num_layers=8, num_kv_heads=8, head_size=64, tp_size=1, dp_size=3, nnodes=2).freeze()
    m.freeze()
    with pytest.raises(Exception):
        m.num_layers = 1


def test_sglang_fp8_latent_cache_with_indexer_has_the_packed_head_width():
    from types import SimpleNamespace as NS
    from flexkv_b200.integration.config import FlexKVConfig
    c = FlexKVConfig()
    c.post_init_from_sglang_config(NS(kv_cache_dtype="fp8_e4m3"),
                                   NS(num_hidden_layers=4, is_mla=True, kv_lora_rank=512, qk_rope_head_dim=64,
                                      index_head_dim=128, dtype=torch.bfloat16), 64)
    assert c.model_config.dtype == torch.float8_e4m3fn and c.model_config.head_size == 512 + 16 + 128
    c = FlexKVConfig()
    c.post_init_from_sglang_config(NS(kv_cache_dtype="auto"),
                                   NS(num_hidden_layers=4, is_mla=True, kv_lora_rank=512, qk_rope_head_dim=64,
                                      dtype=torch.bfloat16), 64)
    assert c.model_config.head_size == 576


def test_response_helpers_keep_the_reference_names_and_values():
    import numpy as np
    from flexkv_b200 import KVResponse, KVResponseStatus
    assert {s.name: s.value for s in KVResponseStatus} == {
        "SUCCESS": "success", "NOTFOUND": "not_found", "UNREADY": "unready", "TIMEOUT": "timeout",
        "CANCELLED": "cancelled", "FAILED": "failed"}
    r = KVResponse(KVResponseStatus.SUCCESS, 3, [np.array([1, 1, 0], bool), np.array([0, 1], bool)])
    assert r.ok and r.num_tokens() == 3 and r.get_mask(1).tolist() == [False, True]
    with pytest.raises(AssertionError):
        r.get_mask(2)
    assert not KVResponse(KVResponseStatus.TIMEOUT, 4, None).ok and not KVResponseStatus.TIMEOUT.terminal


def test_settings_kept_for_compatibility_are_reported_not_ignored_silently():
    from flexkv_b200.common.config import CacheConfig
    assert CacheConfig().settings_without_effect() == []
    c = CacheConfig(enable_ssd=True, enable_nixl=True, num_tmp_cpu_blocks=64, mooncake_config_path="/x.json",
                    enable_3rd_remote=True, distributed_node_id=3, local_zmq_port=6000)
    assert c.enable_gds is True                     # NIXL's role (SSD <-> GPU) is served by the GDS worker
    names = [n for n, _ in c.settings_without_effect()]
    assert names == ["enable_nixl", "use_hugepage_tmp_buffer / num_tmp_cpu_blocks",
                     "mooncake_config_path / mooncake_store_config_path",
                     "distributed_node_id", "local_zmq_ip / local_zmq_port"]
    assert c.enable_kv_sharing and c.enable_remote        # enable_3rd_remote: the shared remote tier is on
    c = CacheConfig(enable_3rd_remote=True, use_mooncake_store_backend=True)
    assert [n for n, _ in c.settings_without_effect()] == ["enable_3rd_remote"]


def test_a_deployment_file_written_for_the_reference_loads(tmp_path):
    """Every key of the reference's user configuration is accepted; the ones that have no effect here are named
    by ``settings_without_effect`` instead of failing the start-up."""
    import json
    from flexkv_b200.common.config import (CacheConfig, ModelConfig, load_user_config_from_file,
                                          update_default_config_from_user_config)
    f = tmp_path / "flexkv.json"
    f.write_text(json.dumps(dict(cpu_cache_gb=4, ssd_cache_gb=8, ssd_cache_dir=str(tmp_path), enable_gds=False,
                                 enable_nixl=True, use_hugepage_cpu_buffer=False, enable_p2p_cpu=True,
                                 enable_p2p_ssd=True, enable_3rd_remote=False, use_mooncake_store_backend=False,
                                 mooncake_store_config_path="/etc/mc.json", local_zmq_ip="10.0.0.5",
                                 local_zmq_port=6001, redis_host="10.0.0.9", redis_port=6380, redis_password="x",
                                 local_ip="10.0.0.5", node_ttl_seconds=45, kv_cache_dtype="bf16",
                                 swa_multi_group=False)))
    u = load_user_config_from_file(str(f))
    assert u.overrides == {}
    m = ModelConfig(num_layers=4, num_kv_heads=2, head_size=64)
    c = CacheConfig(tokens_per_block=16)
    update_default_config_from_user_config(m, c, u)
    assert c.enable_ssd and c.enable_p2p_ssd and c.enable_gds            # enable_nixl -> the GDS worker
    assert (c.redis_host, c.redis_port, c.node_ttl_seconds, c.local_zmq_port) == ("10.0.0.9", 6380, 45, 6001)
    assert c._swa_multi_group is False
    names = [n for n, _ in c.settings_without_effect()]
    assert "enable_nixl" in names and "local_zmq_ip / local_zmq_port" in names
    assert "mooncake_config_path / mooncake_store_config_path" in names


def test_layout_takes_the_reference_spelling():
    from flexkv_b200.common.storage import KVCacheLayout, KVCacheLayoutType as LT
    a = KVCacheLayout(type=LT.LAYERFIRST, num_layer=4, num_block=8, tokens_per_block=16, num_head=2, head_size=64, kv_dim=2)
    assert a.kv_dim == 2 and not a.is_mla and a == KVCacheLayout(LT.LAYERFIRST, 4, 8, 16, 2, 64)
    mla = KVCacheLayout(LT.LAYERFIRST, 4, 8, 64, 1, 576, 1)                  # kv_dim as the seventh positional
    assert mla.kv_dim == 1 and mla.is_mla and mla == KVCacheLayout(LT.LAYERFIRST, 4, 8, 64, 1, 576, is_mla=True)
    packed = KVCacheLayout(LT.LAYERFIRST, 4, 8, 16, 8, 72, kv_dim=1, num_kv_heads=8)   # packed 4-D cache: not MLA
    assert packed.kv_dim == 1 and not packed.is_mla and packed.num_kv_heads == 8
    assert packed.div_head(2).num_head == 4 and packed._replace(num_layer=1).kv_dim == 1


def test_environment_spellings_of_the_reference_are_understood(monkeypatch):
    """Deployment scripts written for the reference set these names; each reaches the same knob here."""
    from types import SimpleNamespace as NS
    from flexkv_b200.integration.config import FlexKVConfig
    from flexkv_b200.integration.sglang.comm import layerwise_wait_timeout_s
    from flexkv_b200.storage.storage_engine import host_register_chunk_bytes
    from flexkv_b200.common import memory_handle
    monkeypatch.delenv("FLEXKV_HOST_REGISTER_CHUNK_BYTES", raising=False)
    assert host_register_chunk_bytes() == 0
    monkeypatch.setenv("FLEXKV_CUDAHOST_CHUNK_SIZE_GB", "0.5")
    assert host_register_chunk_bytes() == 1 << 29
    monkeypatch.setenv("FLEXKV_HOST_REGISTER_CHUNK_BYTES", "4096")
    assert host_register_chunk_bytes() == 4096
    assert layerwise_wait_timeout_s() == 240.0
    monkeypatch.setenv("FLEXKV_LAYERWISE_WAIT_TIMEOUT_S", "12.5")
    assert layerwise_wait_timeout_s() == 12.5
    monkeypatch.setenv("FLEXKV_LAYERWISE_WAIT_TIMEOUT_S", "soon")
    assert layerwise_wait_timeout_s() == 240.0
    monkeypatch.delenv("FLEXKV_VMM_FD_DIR", raising=False)
    monkeypatch.setenv("FLEXKV_VMM_FD_SOCK_DIR", "/run/x")
    assert memory_handle.fd_server_path(77).startswith("/run/x/")
    monkeypatch.setenv("FLEXKV_MASTER_HOST", "10.0.0.7")
    monkeypatch.setenv("FLEXKV_MASTER_PORTS", "7001, 7002,7003")
    cfg = FlexKVConfig()
    model = NS(num_hidden_layers=2, num_key_value_heads=2, head_dim=16, dtype="bfloat16")
    cfg.post_init_from_sglang_config(NS(kv_cache_dtype="auto"), model, page_size=16)
    assert cfg.model_config.master_host == "10.0.0.7" and cfg.model_config.master_ports == ("7001", "7002", "7003")
    monkeypatch.setenv("FLEXKV_MASTER_PORTS", "7001")
    with pytest.raises(ValueError, match="three"):
        FlexKVConfig().post_init_from_sglang_config(NS(kv_cache_dtype="auto"), model, page_size=16)
