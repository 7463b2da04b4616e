"""Caches made of several layer groups with different KV shapes: byte-flat host blocks with
per-group offsets, one registration per (rank, group), shared block ids
(reference format: flexkv/common/storage.py:87-127,249-286; tests test_config_swa_multi_group.py,
test_layerwise_multi_group_swa.py for the format)."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.common.config import LayerGroupSpec, ModelConfig
from flexkv_b200.common.storage import KVCacheLayout, KVCacheLayoutType

T = 8


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def _alloc(num_layers, kv_dim, nb, tokens, heads, head, dtype, dev, seed):
    g = torch.Generator().manual_seed(seed)
    shape = (kv_dim, nb, tokens, heads, head) if kv_dim == 2 else (nb, tokens, heads * head)
    ts = [torch.randn(*shape, generator=g).to(dtype).to(dev) for _ in range(num_layers)]
    lay = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, num_layers, nb, tokens, heads, head, is_mla=(kv_dim == 1))
    return ts, lay


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_two_groups_round_trip(device):
    dev = "cpu" if device == "cpu" else torch.device(device)
    # group 0: 3 full-attention layers, K and V, 2 heads x 16; group 1: 2 compressed layers that keep one
    # latent of 24 values for every 4th token (T / 4 tokens per block)
    groups = [LayerGroupSpec(3, 2, 16, kv_dim=2, name="full"),
              LayerGroupSpec(2, 1, 24, kv_dim=1, compress_ratio=4, name="latent")]
    model = ModelConfig(num_layers=5, num_kv_heads=2, head_size=16, dtype=torch.bfloat16, layer_groups=groups)
    mgr = KVManager(model, CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    NB = 32
    g0, lay0 = _alloc(3, 2, NB, T, 2, 16, torch.bfloat16, dev, 1)
    g1, lay1 = _alloc(2, 1, NB, T // 4, 1, 24, torch.bfloat16, dev, 2)
    mgr.register_gpu_tensors(g0, lay0, group_id=0)
    mgr.register_gpu_tensors(g1, lay1, group_id=1)
    mgr.start(); mgr.wait_ready(30)
    try:
        host = mgr.transfer_manager.storage.host
        per_block = 3 * 2 * T * 2 * 16 * 2 + 2 * 1 * (T // 4) * 24 * 2
        assert host.block_bytes == per_block and host.layout.groups[1].offset_bytes == 3 * 2 * T * 2 * 16 * 2
        tok = np.arange(4 * T, dtype=np.int64)
        src, dst = [3, 9, 1, 30], [20, 21, 22, 23]
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want0 = [t[:, src].clone() for t in g0]
        want1 = [t[src].clone() for t in g1]
        for t in g0:
            t[:, dst] = 0
        for t in g1:
            t[dst] = 0
        tid = mgr.get_async(tok, slots(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(3):
            assert torch.equal(g0[l][:, dst], want0[l])
        for l in range(2):
            assert torch.equal(g1[l][dst], want1[l])
    finally:
        mgr.shutdown()


def test_missing_group_registration_is_reported():
    groups = [LayerGroupSpec(1, 1, 8, kv_dim=1), LayerGroupSpec(1, 1, 16, kv_dim=1)]
    model = ModelConfig(num_layers=2, num_kv_heads=1, head_size=8, dtype=torch.bfloat16, layer_groups=groups)
    mgr = KVManager(model, CacheConfig(tokens_per_block=T, num_cpu_blocks=4), require_gpu=True)
    a, la = _alloc(1, 1, 8, T, 1, 8, torch.bfloat16, "cpu", 1)
    mgr.register_gpu_tensors(a, la, group_id=0)
    mgr.register_gpu_tensors(a, la, group_id=0)       # the second group never arrives
    mgr.start()
    try:
        with pytest.raises((RuntimeError, TimeoutError)):
            mgr.wait_ready(5)
    finally:
        mgr.shutdown()


def test_one_call_registration_of_every_group_through_the_tp_client():
    """The registration form of engine integrations written for the reference: one ``register_to_server`` call
    carries every layer group (``handles_per_group`` / ``gpu_layouts``), the spec list travels with it, and an
    ``override_device_id`` replaces the client's device id (flexkv/server/client.py:366-470)."""
    from flexkv_b200 import KVTPClient
    from flexkv_b200.server.utils import unique_ipc_endpoint
    groups = [LayerGroupSpec(3, 2, 16, kv_dim=2, name="full", layer_indices=[0, 2, 4]),
              LayerGroupSpec(2, 1, 24, kv_dim=1, compress_ratio=4, name="latent", layer_indices=[1, 3])]
    assert groups[0].layer_ids == [0, 2, 4]
    model = ModelConfig(num_layers=5, num_kv_heads=2, head_size=16, dtype=torch.bfloat16)     # groups arrive later
    reg = unique_ipc_endpoint("reg")
    mgr = KVManager(model, CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True, gpu_register_port=reg)
    NB = 32
    g0, lay0 = _alloc(3, 2, NB, T, 2, 16, torch.bfloat16, "cpu", 1)
    g1, lay1 = _alloc(2, 1, NB, T // 4, 1, 24, torch.bfloat16, "cpu", 2)
    mgr.start()
    client = KVTPClient(reg, dp_client_id=0, device_id=7)
    client.register_to_server(g0 + g1, lay0, mode="same_process", layer_groups=groups, gpu_layouts=[lay0, lay1],
                              handles_per_group=[g0, g1], override_device_id=0)
    assert client.device_id == 0
    try:
        mgr.wait_ready(30)
        assert len(mgr.transfer_manager.model_config.layer_groups) == 2
        tok = np.arange(4 * T, dtype=np.int64)
        src, dst = [3, 9, 1, 30], [20, 21, 22, 23]
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want1 = [t[src].clone() for t in g1]
        for t in g1:
            t[dst] = 0
        tid = mgr.get_async(tok, slots(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(g1[l][dst], want1[l])
        with pytest.raises(ValueError, match="go together"):
            client.register_to_server(g0, lay0, swa_layer_groups=[1], swa_gpu_layouts=None, swa_handles_per_group=None)
    finally:
        client.shutdown()
        mgr.shutdown()
