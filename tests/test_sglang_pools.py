"""SGLang KV pool objects made of several parts (indexer keys, split compressed pools, a sliding-window pool
with compressor-state sidecars): resolution into layer groups and window geometry, registration of every part
through the connector, and a store / lookup / load round trip of all of it on CPU
(reference behaviour: flexkv/integration/sglang/connector.py:1599-1897; tests test_config_swa_multi_group.py,
test_layerwise_dsv4_multi_group_swa_roundtrip.py)."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.common.config import ModelConfig
from flexkv_b200.integration.config import FlexKVConfig
from flexkv_b200.integration.sglang.connector import FlexKVConnector
from flexkv_b200.integration.sglang.pools import (build_swa_slot_mapping, layer_group_specs, resolve_kv_pool,
                                                  window_pool_config)
from flexkv_b200.server.utils import unique_ipc_endpoint

T = 128          # page size in tokens (the c128 group stores one token per page)
NP = 16          # pages per pool


def _rand(shape, seed, dtype=torch.uint8):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, shape, dtype=torch.uint8, generator=g).view(dtype)


class _Pool:
    def __init__(self, layers, sub_page, bytes_per_token, seed):
        self.page_size = sub_page
        self._bpt = bytes_per_token
        self.kv_buffer = [_rand((NP, sub_page * bytes_per_token), seed + i) for i in range(layers)]

    def get_bytes_per_token(self):
        return self._bpt


class _Indexer:
    def __init__(self, layers, sub_page, bytes_per_token, seed):
        self.page_size = sub_page
        self.index_k_with_scale_buffer = [_rand((NP, sub_page * bytes_per_token), seed + i) for i in range(layers)]


class _Score:
    def __init__(self, t):
        self.kv_score = t


class _State:
    def __init__(self, ring, width, seed):
        self.ring_size = ring
        self.kv_score_buffer = _Score(_rand((NP * ring, width), seed))


class SplitKV:
    """Four model layers: 0 and 2 keep every 4th token (plus indexer keys and compressor state), 1 and 3 every
    128th; every layer has sliding-window KV."""

    def __init__(self):
        self.compression_ratios = [4, 128, 4, 128]
        self.c4_kv_pool = _Pool(2, T // 4, 8, 10)
        self.c128_kv_pool = _Pool(2, T // 128, 16, 20)
        self.c4_indexer_kv_pool = _Indexer(2, T // 4, 4, 30)
        self.swa_kv_pool = _Pool(4, T, 4, 40)
        self.swa_page_size = T
        self.compress_state_pools = [_State(32, 8, 50), None, _State(32, 8, 51), None]
        self.indexer_compress_state_pools = [_State(32, 4, 60), None, _State(32, 4, 61), None]

    def translate_loc_from_full_to_swa(self, idx):
        return idx.clone()                      # the window pool mirrors the full pool's page numbering here

    def parts(self):
        out = self.c4_kv_pool.kv_buffer + self.c128_kv_pool.kv_buffer + \
            self.c4_indexer_kv_pool.index_k_with_scale_buffer + self.swa_kv_pool.kv_buffer
        for pools in (self.compress_state_pools, self.indexer_compress_state_pools):
            out += [p.kv_score_buffer.kv_score.view(NP, -1) for p in pools if p is not None]
        return out


def test_split_pool_resolves_into_groups_window_and_sidecars():
    kv = SplitKV()
    pool = resolve_kv_pool(kv, T)
    assert pool.kind == "split" and [g.name for g in pool.groups] == ["c4", "c128", "c4_indexer"]
    assert [g.layer_ids for g in pool.groups] == [[0, 2], [1, 3], [0, 2]]
    specs = layer_group_specs(pool, T)
    assert [(s.num_layers, s.head_size, s.compress_ratio, s.kv_dim) for s in specs] == \
        [(2, 8, 4, 1), (2, 16, 128, 1), (2, 4, 4, 1)]
    assert [s.layer_ids for s in specs] == [[0, 2], [1, 3], [0, 2]]
    assert len(pool.swa_buffers) == 4 and [g.name for g in pool.state_groups] == ["c4_attention_state",
                                                                                  "c4_indexer_state"]
    swa = window_pool_config(pool, T)
    assert swa.enabled and swa.num_swa_layers == 4 and swa.bytes_per_token_per_layer == 4
    assert swa.sidecar_groups == [(2, 32 * 8), (2, 32 * 4)] and swa.wait_for_registration
    assert resolve_kv_pool(kv, T, include_state=False).state_groups == []
    # a later pipeline stage sees its own layers, numbered from zero
    kv._stage_start, kv._stage_end = 2, 4
    kv.c4_kv_pool.kv_buffer = kv.c4_kv_pool.kv_buffer[:1]
    kv.c128_kv_pool.kv_buffer = kv.c128_kv_pool.kv_buffer[:1]
    kv.c4_indexer_kv_pool.index_k_with_scale_buffer = kv.c4_indexer_kv_pool.index_k_with_scale_buffer[:1]
    assert [g.layer_ids for g in resolve_kv_pool(kv, T).groups] == [[0], [1], [0]]


def test_window_slot_mapping_keeps_the_mapped_tail():
    class KV:
        swa_kv_pool = object()

        @staticmethod
        def translate_loc_from_full_to_swa(idx):
            out = idx.clone()
            out[:5] = 0                          # these tokens slid out of the window
            return out
    full = torch.arange(100, 112)
    assert build_swa_slot_mapping(KV, full).tolist() == list(range(105, 112))
    KV.translate_loc_from_full_to_swa = staticmethod(lambda idx: torch.zeros_like(idx))
    assert build_swa_slot_mapping(KV, full) is None
    assert build_swa_slot_mapping(object(), full) is None


def test_plain_pool_with_indexer_keys_becomes_two_groups():
    class KV:
        k_buffer = [torch.zeros(NP * 8, 2, 16, dtype=torch.bfloat16) for _ in range(3)]
        v_buffer = [torch.zeros(NP * 8, 2, 16, dtype=torch.bfloat16) for _ in range(3)]
        index_k_with_scale_buffer = [torch.zeros(NP, 8 * 12, dtype=torch.uint8) for _ in range(3)]
    pool = resolve_kv_pool(KV, 8)
    assert pool.kind == "indexer"
    specs = layer_group_specs(pool, 8)
    assert [(s.num_layers, s.num_kv_heads, s.head_size, s.kv_dim, s.dtype) for s in specs] == \
        [(3, 2, 16, 2, torch.bfloat16), (3, 1, 12, 1, torch.uint8)]

    class Plain:
        kv_buffer = [torch.zeros(NP * 8, 1, 64) for _ in range(2)]
    assert layer_group_specs(resolve_kv_pool(Plain, 8), 8) is None
    with pytest.raises(AttributeError):
        resolve_kv_pool(object(), 8)


def test_connector_round_trip_of_every_part_of_a_split_pool():
    kv = SplitKV()
    cfg = FlexKVConfig()
    cfg.model_config = ModelConfig(num_layers=4, num_kv_heads=1, head_size=16, dtype=torch.uint8, use_mla=True)
    cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=16)
    cfg.gpu_register_port = unique_ipc_endpoint("sgpool")
    cfg.server_recv_port = unique_ipc_endpoint("sgsrv")
    pool = FlexKVConnector.configure_for_pool(cfg, kv, T)
    assert len(cfg.model_config.layer_groups) == 3 and cfg.cache_config.swa.sidecar_groups
    cfg.cache_config.swa.num_slots = 4
    # require_gpu: start-up waits for every registration although the "GPU" tensors are host stand-ins here
    mgr = KVManager(cfg.model_config, cfg.cache_config, require_gpu=True, gpu_register_port=cfg.gpu_register_port)
    mgr.start()
    conn = FlexKVConnector(cfg, page_size=T, kv_manager=mgr)
    try:
        conn.register_kv_pool(kv, pool)
        conn.wait_ready(60)
        host = conn.mgr.transfer_manager.storage.host
        assert host.block_bytes == 2 * 32 * 8 + 2 * 1 * 16 + 2 * 32 * 4
        src, dst = np.array([3, 9]), np.array([12, 5])
        tok = list(range(1000, 1000 + 2 * T))
        slot = np.repeat(src, T) * T + np.tile(np.arange(T), 2)
        saved = [t.clone() for t in kv.parts()]
        assert conn.store_kv("r1", tok, slot) == 2 * T
        assert conn.wait_store("r1")
        for t in kv.parts():
            t[dst] = 0
        assert conn.lookup_kv("r2", tok) == 2 * T
        assert conn.retrieve_kv("r2", np.repeat(dst, T) * T + np.tile(np.arange(T), 2)) == 2 * T
        parts = kv.parts()
        for i in range(6):                                   # c4, c128, indexer: both pages of the sequence
            assert torch.equal(parts[i][dst], saved[i][src]), i
        for i in range(6, len(parts)):                       # window KV and state: the page of the sequence end
            assert torch.equal(parts[i][dst[-1]], saved[i][src[-1]]), i
            assert not parts[i][dst[0]].any()
    finally:
        conn.shutdown()


def test_window_data_plane_follows_the_deployment_switch(monkeypatch):
    """A pool with window layers turns the window data plane on unless FLEXKV_ENABLE_SWA_TRANSFER=0; switched
    off, the geometry stays configured and nothing else forces it back on (reference: tests/test_swa_config_gate.py)."""
    def configured():
        cfg = FlexKVConfig()
        cfg.model_config = ModelConfig(num_layers=4, num_kv_heads=1, head_size=16, dtype=torch.uint8, use_mla=True)
        cfg.cache_config = CacheConfig(tokens_per_block=T, num_cpu_blocks=16)
        FlexKVConnector.configure_for_pool(cfg, SplitKV(), T)
        return cfg.cache_config
    monkeypatch.delenv("FLEXKV_ENABLE_SWA_TRANSFER", raising=False)
    cc = configured()
    assert cc.swa.enabled and cc.enable_swa_transfer is True
    monkeypatch.setenv("FLEXKV_ENABLE_SWA_TRANSFER", "1")
    assert configured().enable_swa_transfer is True
    monkeypatch.setenv("FLEXKV_ENABLE_SWA_TRANSFER", "0")
    cc = configured()
    assert cc.swa.enabled and cc.enable_swa_transfer is False
