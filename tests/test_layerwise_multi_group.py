"""Layerwise restore of caches made of several layer groups: which (group, layer) pairs make up
a model layer (CPU), and on a GPU the bytes, one eventfd unit per MODEL layer after all of its
members have landed, member-less layers, and the whole path through KVManager.launch
(reference: csrc/layerwise.cpp:1313-1682, tests/test_layerwise_multi_group_swa.py)."""
import os
import struct

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager, _native
from flexkv_b200.common.config import GLOBAL_CONFIG_FROM_ENV, LayerGroupSpec, ModelConfig
from flexkv_b200.common.storage import GroupLayout, KVCacheLayout, KVCacheLayoutType
from flexkv_b200.storage.gpu_layout import register_tensors
from flexkv_b200.transfer.layerwise import layer_members

T = 8
C = _native.C


def _groups():
    return [GroupLayout(3, 2, T, 2, 16, 2), GroupLayout(2, 1, T // 4, 1, 24, 2)]


def test_members_follow_layer_ids_or_pair_up_from_layer_zero():
    g = _groups()
    m = ModelConfig(num_layers=3, num_kv_heads=2, head_size=16, dtype=torch.bfloat16,
                    layer_groups=[LayerGroupSpec(3, 2, 16), LayerGroupSpec(2, 1, 24, kv_dim=1, compress_ratio=4)])
    assert layer_members(m, g) == [[(0, 0), (1, 0)], [(0, 1), (1, 1)], [(0, 2)]]
    m = ModelConfig(num_layers=6, num_kv_heads=2, head_size=16, dtype=torch.bfloat16,
                    layer_groups=[LayerGroupSpec(3, 2, 16, layer_ids=[0, 2, 5]),
                                  LayerGroupSpec(2, 1, 24, kv_dim=1, compress_ratio=4, layer_ids=[5, 1])])
    assert layer_members(m, g) == [[(0, 0)], [(1, 1)], [(0, 1)], [], [], [(0, 2), (1, 0)]]
    bad = ModelConfig(num_layers=3, num_kv_heads=2, head_size=16, dtype=torch.bfloat16,
                      layer_groups=[LayerGroupSpec(3, 2, 16, layer_ids=[0, 1]), LayerGroupSpec(2, 1, 24)])
    with pytest.raises(ValueError):
        layer_members(bad, g)


def _alloc(num_layers, kv_dim, nb, tokens, heads, head, dev, seed):
    g = torch.Generator().manual_seed(seed)
    shape = (kv_dim, nb, tokens, heads, head) if kv_dim == 2 else (nb, tokens, heads * head)
    ts = [torch.randn(*shape, generator=g).to(torch.bfloat16).to(dev) for _ in range(num_layers)]
    lay = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, num_layers, nb, tokens, heads, head, is_mla=(kv_dim == 1))
    return ts, lay


def _drain(fd):
    n = 0
    while True:
        try:
            n += struct.unpack("Q", os.read(fd, 8))[0]
        except BlockingIOError:
            return n


def _host_block(pool, b, groups):
    """The expected bytes of host block ``b`` split per (group, layer, kv)."""
    out = {}
    for gid, g in enumerate(groups):
        for l in range(g.num_layers):
            for k in range(g.kv_dim):
                off = g.offset_bytes + l * g.layer_stride_bytes + k * g.chunk_bytes
                out[(gid, l, k)] = pool[b, off:off + g.chunk_bytes]
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("notify", ["hostfunc", "polling", "flag"])
def test_native_group_restores_members_and_signals_model_layers(notify):
    dev = torch.device("cuda:0")
    NB = 32
    groups = _groups()
    KVCacheLayout(KVCacheLayoutType.BLOCKFIRST, 5, NB, T, 2, 16, groups=groups)        # fills the offsets
    block_bytes = sum(g.bytes for g in groups)
    g0, lay0 = _alloc(3, 2, NB, T, 2, 16, dev, 1)
    g1, lay1 = _alloc(2, 1, NB, T // 4, 1, 24, dev, 2)
    regs = [register_tensors(g0, lay0), register_tensors(g1, lay1)]
    gen = torch.Generator().manual_seed(9)
    pool = torch.randint(0, 256, (NB, block_bytes), dtype=torch.uint8, generator=gen).pin_memory()
    # model layers: 0 = (g0 l0, g1 l1), 1 = nothing, 2 = (g0 l1), 3 = (g1 l0, g0 l2)
    members = [[(0, 0), (1, 1)], [], [(0, 1)], [(1, 0), (0, 2)]]
    native_groups = [dict(gpus=[regs[i].as_native()],
                          host=dict(base=pool.data_ptr() + g.offset_bytes, layer_stride=g.layer_stride_bytes,
                                    kv_stride=g.chunk_bytes, block_stride=block_bytes, num_blocks=NB),
                          options=dict(num_layers=g.num_layers, kv_dim=g.kv_dim, chunk_bytes=g.chunk_bytes,
                                       shared_kv=True))
                     for i, g in enumerate(groups)]
    opts = dict(num_layers=len(members), kv_dim=1, chunk_bytes=16, max_blocks_per_op=NB, notify_mode=notify,
                num_counters=2, layers_per_batch=1, h2d=dict(num_ctas=4, tile_bytes=8192, engine=0))
    host = dict(base=pool.data_ptr(), layer_stride=block_bytes, kv_stride=0, block_stride=block_bytes, num_blocks=NB)
    grp = C.LayerwiseGroup.multi_group(native_groups, members, host, opts)
    assert grp.is_multi_group and grp.num_layers == 4
    rng = np.random.default_rng(4)
    n = 11
    cpu = rng.permutation(NB)[:n].astype(np.int64)
    for counter in (1, 0):
        fds = [grp.eventfd_of(counter, 0, l) for l in range(4)]
        assert all(_drain(fd) == 0 for fd in fds)
        dst = rng.permutation(NB)[:n].astype(np.int64)
        r = grp.restore(dst, cpu, counter)
        assert r.status == 0 and len(r.layer_done_ms) == 4
        assert all(b >= a for a, b in zip(r.layer_done_ms, r.layer_done_ms[1:]))
        assert [_drain(fd) for fd in fds] == [1, 1, 1, 1]            # the member-less layer fires too
        for i in range(n):
            want = _host_block(pool, int(cpu[i]), groups)
            for l in range(3):
                for k in range(2):
                    got = g0[l][k, int(dst[i])].contiguous().view(torch.uint8).reshape(-1).cpu()
                    assert torch.equal(got, want[(0, l, k)])
            for l in range(2):
                got = g1[l][int(dst[i])].contiguous().view(torch.uint8).reshape(-1).cpu()
                assert torch.equal(got, want[(1, l, 0)])
        import ctypes
        ep = grp.epoch_of(counter)
        assert list((ctypes.c_uint32 * 4).from_address(grp.host_flags_ptr(0, counter))) == [ep] * 4
    e = np.zeros(0, dtype=np.int64)
    assert grp.restore(e, e, 0).status == 0                           # empty restore releases every layer
    assert [_drain(grp.eventfd_of(0, 0, l)) for l in range(4)] == [1, 1, 1, 1]
    # a group layer that belongs to no model layer would never be restored: refused at construction
    with pytest.raises(ValueError):
        C.LayerwiseGroup.multi_group(native_groups, [[(0, 0)], [(0, 1), (1, 0)]], host, opts)


def _slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


@pytest.mark.gpu
@pytest.mark.parametrize("multi", [False, True])
def test_layerwise_launch_through_the_manager(multi, monkeypatch):
    """put, then a batched get launched with layerwise_transfer=True: bytes are exact and every model layer's
    eventfd of the chosen counter carries exactly one unit."""
    monkeypatch.setattr(GLOBAL_CONFIG_FROM_ENV, "enable_layerwise_transfer", True)
    dev = torch.device("cuda:0")
    NB = 32
    if multi:
        specs = [LayerGroupSpec(3, 2, 16, kv_dim=2, name="full"),
                 LayerGroupSpec(2, 1, 24, kv_dim=1, compress_ratio=4, name="latent", layer_ids=[0, 2])]
        model = ModelConfig(num_layers=3, num_kv_heads=2, head_size=16, dtype=torch.bfloat16, layer_groups=specs)
    else:
        model = ModelConfig(num_layers=3, num_kv_heads=2, head_size=16, dtype=torch.bfloat16)
    mgr = KVManager(model, CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    g0, lay0 = _alloc(3, 2, NB, T, 2, 16, dev, 1)
    g1, lay1 = _alloc(2, 1, NB, T // 4, 1, 24, dev, 2)
    if multi:
        mgr.register_gpu_tensors(g0, lay0, group_id=0)
        mgr.register_gpu_tensors(g1, lay1, group_id=1)
    else:
        mgr.register_gpu_tensors(g0, lay0)
    mgr.start(); mgr.wait_ready(30)
    try:
        from flexkv_b200.common.transfer import TransferType
        workers = mgr.transfer_manager.engine._workers
        lw = [w for (k, t), w in workers.items() if t == TransferType.LAYERWISE]
        assert len(lw) == 1 and lw[0].group.is_multi_group == multi and lw[0].group.num_layers == 3
        tok = np.arange(4 * T, dtype=np.int64)
        src, dst = [3, 9, 1, 30], [20, 21, 22, 23]
        tid = mgr.put_async(tok, _slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want0 = [t[:, src].clone() for t in g0]
        want1 = [t[src].clone() for t in g1]
        for t in g0:
            t[:, dst] = 0
        for t in g1:
            t[dst] = 0
        tid, mask = mgr.get_match(tok)
        assert mask.sum() == 4 * T
        fds = [lw[0].group.eventfd_of(2, 0, l) for l in range(3)]
        assert all(_drain(fd) == 0 for fd in fds)
        (bid,) = mgr.launch([tid], [_slots(dst)], as_batch=True, layerwise_transfer=True, counter_id=2)
        assert mgr.wait(bid)[bid].status.value == "success"
        assert [_drain(fd) for fd in fds] == [1, 1, 1]
        for l in range(3):
            assert torch.equal(g0[l][:, dst], want0[l])
        if multi:
            for l in range(2):
                assert torch.equal(g1[l][dst], want1[l])
    finally:
        mgr.shutdown()
