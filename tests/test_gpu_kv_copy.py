"""Paged gather/scatter kernels against a plain PyTorch reference of the same
move (index_select / index_copy on the paged tensors and the host pool viewed
as a tensor), byte for byte, across engine layouts, host layouts, engines and
awkward sizes."""
import numpy as np
import pytest
import torch

from flexkv_b200.models import KVShape, alloc_paged_cache
from flexkv_b200.ops.kv_copy import (ENGINE_SIMT, ENGINE_TMA, HostSide, decode_status, kv_copy, kv_copy_refshape,
                                     new_status)
from flexkv_b200.storage.gpu_layout import register_tensors

pytestmark = pytest.mark.gpu


def _host_pool(shape: KVShape, num_blocks: int, tp: int = 1):
    """BLOCKFIRST pinned pool [B][L][K][chunk] as uint8."""
    H = shape.num_kv_heads if shape.use_mla else shape.num_kv_heads // tp
    chunk = shape.tokens_per_block * H * shape.head_size * shape.dtype.itemsize
    pool = torch.zeros(num_blocks, shape.num_layers, shape.kv_dim, chunk, dtype=torch.uint8).pin_memory()
    side = HostSide(pool.data_ptr(), shape.kv_dim * chunk, chunk, shape.num_layers * shape.kv_dim * chunk, num_blocks)
    return pool, side, chunk


def _gpu_chunk(tensors, layout_name, shape, layer, kv, block, layerblock=False):
    """uint8 view of the chunk (layer, kv, block) inside the engine's tensors."""
    if layout_name == "vllm":
        t = tensors[layer]
        if shape.use_mla:
            c = t[block]
        elif layerblock:
            c = t[block, kv]
        else:
            c = t[kv, block]
    elif layout_name == "sglang":
        c = tensors[kv * shape.num_layers + layer][block] if shape.kv_dim == 2 else tensors[layer][block]
    else:
        c = tensors[0][block, layer, kv]
    return c.contiguous().view(torch.uint8).reshape(-1)


CASES = [
    ("vllm", False, KVShape("a", 3, 4, 32, tokens_per_block=16)),
    ("vllm", True, KVShape("b", 2, 2, 64, tokens_per_block=8)),
    ("sglang", False, KVShape("c", 4, 2, 32, tokens_per_block=16)),
    ("trtllm", False, KVShape("d", 3, 2, 16, tokens_per_block=4)),
    ("vllm", False, KVShape("mla", 3, 1, 576, use_mla=True, tokens_per_block=64)),
    ("vllm", False, KVShape("odd", 2, 1, 585, dtype=torch.uint8, use_mla=True, tokens_per_block=8)),  # 4680 B chunks
    ("sglang", False, KVShape("deep", 136, 2, 16, tokens_per_block=4)),      # 272 tensors: table in device memory
]


@pytest.mark.parametrize("engine", [ENGINE_TMA, ENGINE_SIMT])
@pytest.mark.parametrize("layout_name,layerblock,shape", CASES)
def test_roundtrip_matches_torch(layout_name, layerblock, shape, engine):
    dev = torch.device("cuda:0")
    NG, NC, n = 37, 29, 17
    tensors, layout = alloc_paged_cache(shape, NG, dev, layout_name, layerblock=layerblock,
                                        fill="normal", seed=1)
    reg = register_tensors(tensors, layout)
    pool, side, chunk = _host_pool(shape, NC)
    assert reg.chunk_bytes == chunk
    rng = np.random.default_rng(0)
    g = rng.permutation(NG)[:n].astype(np.int64)
    c = rng.permutation(NC)[:n].astype(np.int64)
    status = new_status(dev)
    keep = kv_copy(reg, side, g, c, h2d=False, engine=engine, num_ctas=5, tile_bytes=2048, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    for i in range(n):
        for l in range(shape.num_layers):
            for k in range(shape.kv_dim):
                ref = _gpu_chunk(tensors, layout_name, shape, l, k, int(g[i]), layerblock).cpu()
                assert torch.equal(pool[int(c[i]), l, k], ref), (i, l, k)
    # untouched host blocks stay zero
    mask = torch.ones(NC, dtype=torch.bool)
    mask[torch.from_numpy(c)] = False
    assert int(pool[mask].abs().sum()) == 0

    # restore into different blocks of a zeroed cache
    saved = [t.clone() for t in tensors]
    for t in tensors:
        t.zero_()
    g2 = rng.permutation(NG)[:n].astype(np.int64)
    keep += kv_copy(reg, side, g2, c, h2d=True, engine=engine, num_ctas=3, tile_bytes=4096, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    for i in range(n):
        for l in range(shape.num_layers):
            for k in range(shape.kv_dim):
                want = _gpu_chunk(saved, layout_name, shape, l, k, int(g[i]), layerblock)
                got = _gpu_chunk(tensors, layout_name, shape, l, k, int(g2[i]), layerblock)
                assert torch.equal(want, got), (i, l, k)


def test_layer_range_and_device_ids():
    dev = torch.device("cuda:0")
    shape = KVShape("r", 6, 2, 32, tokens_per_block=16)
    tensors, layout = alloc_paged_cache(shape, 16, dev, "vllm", fill="normal", seed=3)
    reg = register_tensors(tensors, layout)
    pool, side, chunk = _host_pool(shape, 16)
    g = torch.tensor([3, 1, 7], dtype=torch.int64, device=dev)        # ids resident on the device
    c = torch.tensor([0, 5, 2], dtype=torch.int64, device=dev)
    kv_copy(reg, side, g, c, h2d=False, layer_start=2, num_layers=3)
    torch.cuda.synchronize()
    for l in range(6):
        for i in range(3):
            ref = tensors[l][:, int(g[i])].contiguous().view(torch.uint8).reshape(2, -1).cpu()
            if 2 <= l < 5:
                assert torch.equal(pool[int(c[i]), l], ref)
            else:
                assert int(pool[int(c[i]), l].abs().sum()) == 0


def test_out_of_range_ids_are_reported_not_followed():
    dev = torch.device("cuda:0")
    shape = KVShape("e", 2, 2, 32, tokens_per_block=16)
    tensors, layout = alloc_paged_cache(shape, 8, dev, "vllm", fill="normal", seed=4)
    reg = register_tensors(tensors, layout)
    pool, side, chunk = _host_pool(shape, 8)
    status = new_status(dev)
    g = np.array([1, 99, 2], dtype=np.int64)     # 99 is outside the GPU pool
    c = np.array([0, 1, 77], dtype=np.int64)     # 77 is outside the host pool
    for engine in (ENGINE_TMA, ENGINE_SIMT):
        pool.zero_()
        status.zero_()
        kv_copy(reg, side, g, c, h2d=False, engine=engine, status=status)
        torch.cuda.synchronize()
        assert decode_status(status) == 1 | 2
        assert int(pool[1].abs().sum()) == 0       # the bad pairs were skipped
        ref = tensors[0][:, 1].contiguous().view(torch.uint8).reshape(2, -1).cpu()
        assert torch.equal(pool[0, 0], ref)        # the good pair moved


def test_refshape_baseline_kernel_moves_the_same_bytes():
    dev = torch.device("cuda:0")
    shape = KVShape("f", 4, 2, 64, tokens_per_block=16)
    tensors, layout = alloc_paged_cache(shape, 32, dev, "vllm", fill="normal", seed=5)
    reg = register_tensors(tensors, layout)
    pool, side, _ = _host_pool(shape, 32)
    pool2, side2, _ = _host_pool(shape, 32)
    g = np.arange(20, dtype=np.int64)[::-1].copy()
    c = np.arange(20, dtype=np.int64)
    kv_copy(reg, side, g, c, h2d=False)
    kv_copy_refshape(reg, side2, g, c, h2d=False)
    torch.cuda.synchronize()
    assert torch.equal(pool, pool2)


def test_large_transfer_exceeds_l2_and_is_exact():
    """~256 MiB through the pipeline with the production launch shape."""
    dev = torch.device("cuda:0")
    shape = KVShape("g", 8, 8, 128, tokens_per_block=16)     # 512 KiB per block
    NB = 640
    tensors, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=6)
    reg = register_tensors(tensors, layout)
    pool, side, _ = _host_pool(shape, NB)
    rng = np.random.default_rng(1)
    g = rng.permutation(NB)[:512].astype(np.int64)
    c = rng.permutation(NB)[:512].astype(np.int64)
    status = new_status(dev)
    kv_copy(reg, side, g, c, h2d=False, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    saved = [t.clone() for t in tensors]
    for t in tensors:
        t.zero_()
    kv_copy(reg, side, g, c, h2d=True, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    gi = torch.from_numpy(g).to(dev)
    for l in range(shape.num_layers):
        assert torch.equal(tensors[l][:, gi], saved[l][:, gi])
