"""Copy-engine and adaptive routing of the native transfer group against the
TMA kernel and a PyTorch reference of the same move, byte for byte."""
import numpy as np
import pytest
import torch

from flexkv_b200 import _native
from flexkv_b200.models import KVShape, alloc_paged_cache
from flexkv_b200.storage.gpu_layout import register_tensors

pytestmark = pytest.mark.gpu
C = _native.C

ENG = {"tma": 0, "ce": 2, "auto": 3}


def _group(shape, layout_name, NG, NC, dev, reg=None):
    tensors = None
    if reg is None:
        tensors, layout = alloc_paged_cache(shape, NG, dev, layout_name, fill="normal", seed=3)
        reg = register_tensors(tensors, layout)
    chunk = reg.chunk_bytes
    pool = torch.zeros(NC, shape.num_layers, shape.kv_dim, chunk, dtype=torch.uint8).pin_memory()
    host = dict(base=pool.data_ptr(), layer_stride=shape.kv_dim * chunk, kv_stride=chunk,
                block_stride=shape.num_layers * shape.kv_dim * chunk, num_blocks=NC)
    opts = dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim, chunk_bytes=chunk, max_blocks_per_op=4096,
                ce_min_bytes_per_copy=64 << 10)
    grp = C.TransferGroup([reg.as_native()], host, opts)
    return grp, tensors, pool, reg


@pytest.mark.parametrize("layout_name", ["vllm", "sglang", "trtllm"])
@pytest.mark.parametrize("engine", ["ce", "auto"])
def test_contiguous_runs_match_kernel_bytes(layout_name, engine):
    dev = torch.device("cuda:0")
    shape = KVShape("t", 3, 2, 64, tokens_per_block=16)          # 4 KiB chunks
    NG, NC = 96, 80
    grp, tensors, pool, reg = _group(shape, layout_name, NG, NC, dev)
    # two long runs and a few strays
    g = np.concatenate([np.arange(5, 37), np.arange(60, 84), [2, 90, 44]]).astype(np.int64)
    c = np.concatenate([np.arange(10, 42), np.arange(50, 74), [1, 3, 79]]).astype(np.int64)
    before = grp.ce_ops
    r = grp.transfer(g, c, False, 0, shape.num_layers, ENG[engine])
    assert r.status == 0
    if engine == "ce":
        assert grp.ce_ops == before + 1
    want = pool.clone()
    pool.zero_()
    r = grp.transfer(g, c, False, 0, shape.num_layers, ENG["tma"])
    assert r.status == 0
    assert torch.equal(pool, want)                # same bytes as the kernel path
    assert int(want.count_nonzero()) > 0
    # restore into other blocks through the copy engines, read those back through the kernel
    g2 = ((g + 7) % NG).astype(np.int64)
    assert len(set(g2.tolist())) == len(g2)
    r = grp.transfer(g2, c, True, 0, shape.num_layers, ENG[engine])
    assert r.status == 0
    grp2, _, chk, _ = _group(shape, layout_name, NG, NC, dev, reg=reg)
    c2 = np.arange(len(g2), dtype=np.int64)
    r = grp2.transfer(g2, c2, False, 0, shape.num_layers, ENG["tma"])
    assert r.status == 0
    for i, cb in enumerate(c):
        assert torch.equal(chk[i], want[cb])


def test_auto_sends_scattered_ids_to_the_kernel_and_long_runs_to_the_copy_engines():
    dev = torch.device("cuda:0")
    shape = KVShape("t", 2, 2, 128, tokens_per_block=16)         # 8 KiB chunks
    grp, tensors, pool, _ = _group(shape, "vllm", 512, 512, dev)
    rng = np.random.default_rng(1)
    g = rng.permutation(512)[:128].astype(np.int64)
    c = rng.permutation(512)[:128].astype(np.int64)
    n0 = grp.ce_ops
    assert grp.transfer(g, c, False, 0, 2, ENG["auto"]).status == 0
    assert grp.ce_ops == n0                                         # stayed on the kernel
    g = np.arange(100, 356, dtype=np.int64)
    c = np.arange(17, 273, dtype=np.int64)
    assert grp.transfer(g, c, False, 0, 2, ENG["auto"]).status == 0
    assert grp.ce_ops == n0 + 1


def test_bad_ids_are_reported_by_the_copy_engine_path():
    dev = torch.device("cuda:0")
    shape = KVShape("t", 2, 2, 64, tokens_per_block=16)
    grp, tensors, pool, _ = _group(shape, "vllm", 32, 32, dev)
    g = np.array([0, 1, 2, 99], dtype=np.int64)
    c = np.array([4, 5, 6, 7], dtype=np.int64)
    r = grp.transfer(g, c, False, 0, 2, ENG["ce"])
    assert r.status == 1
    assert int(pool[7].count_nonzero()) == 0 and int(pool[4].count_nonzero()) > 0


def test_scattered_pages_with_host_blocks_in_a_row_go_through_the_staging_area():
    """GPU pages scattered, host blocks allocated in runs: the gather kernel fills a device staging buffer in
    host block format and one large copy moves each piece; bytes equal the kernel path in both directions.
    The staging buffers (4 blocks each here) are reused by several pieces and by both runs."""
    dev = torch.device("cuda:0")
    shape = KVShape("t", 3, 2, 128, tokens_per_block=16)          # 8 KiB chunks, 48 KiB blocks
    NG, NC = 256, 200
    tensors, layout = alloc_paged_cache(shape, NG, dev, "vllm", fill="normal", seed=5)
    reg = register_tensors(tensors, layout)
    chunk = reg.chunk_bytes
    pool = torch.zeros(NC, shape.num_layers, shape.kv_dim, chunk, dtype=torch.uint8).pin_memory()
    host = dict(base=pool.data_ptr(), layer_stride=shape.kv_dim * chunk, kv_stride=chunk,
                block_stride=shape.num_layers * shape.kv_dim * chunk, num_blocks=NC)
    opts = dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim, chunk_bytes=chunk, max_blocks_per_op=4096,
                ce_min_bytes_per_copy=96 << 10, ce_staging_blocks=4)     # runs of >= 2 blocks qualify
    grp = C.TransferGroup([reg.as_native()], host, opts)
    rng = np.random.default_rng(8)
    g = rng.permutation(NG)[:30].astype(np.int64)                 # scattered pages
    c = np.concatenate([np.arange(40, 59), np.arange(120, 131)]).astype(np.int64)   # two host runs: 19 and 11 blocks
    n0 = grp.staged_ops
    assert grp.transfer(g, c, False, 0, shape.num_layers, ENG["auto"]).status == 0
    assert grp.staged_ops == n0 + 1
    want = pool.clone()
    pool.zero_()
    assert grp.transfer(g, c, False, 0, shape.num_layers, ENG["tma"]).status == 0
    assert torch.equal(pool, want) and int(want.count_nonzero()) > 0
    # restore through the staging area into other scattered pages
    saved = [t.clone() for t in tensors]
    g2 = rng.permutation(NG)[:30].astype(np.int64)
    assert grp.transfer(g2, c, True, 0, shape.num_layers, ENG["auto"]).status == 0
    assert grp.staged_ops == n0 + 2
    a, b = torch.from_numpy(g).to(dev), torch.from_numpy(g2).to(dev)
    for l in range(shape.num_layers):
        assert torch.equal(tensors[l][:, b], saved[l][:, a])
    # a partial-layer op or a stray host block keeps the op on the kernel
    assert grp.transfer(g, c, False, 0, 2, ENG["auto"]).status == 0
    c3 = c.copy()
    c3[5] = 199
    assert grp.transfer(g, c3, False, 0, shape.num_layers, ENG["auto"]).status == 0
    assert grp.staged_ops == n0 + 2
    # a bad page id is refused on the host: the op falls back to the kernel, which reports it
    gb = g.copy()
    gb[3] = NG + 5
    assert grp.transfer(gb, c, False, 0, shape.num_layers, ENG["auto"]).status == 1
