"""Warm restart of the SSD tier: a second manager on the same cache directories serves the
blocks that the first one wrote, byte for byte; anything that makes the saved image unsafe
(another geometry, a damaged file, a second mount without a clean shutdown in between)
gives a cold start. Index images are also checked natively against the Python index."""
import os

import numpy as np
import pytest
import torch

from flexkv_b200 import _native
from flexkv_b200.cache import persist
from flexkv_b200.cache.mempool import Mempool
from flexkv_b200.cache.radixtree import RadixTreeIndex
from flexkv_b200.models import KVShape

from test_kvmanager_cpu import chunks, slots, start

C = _native.C


def _hashes(rng, n):
    return rng.integers(1, 2**63, size=n, dtype=np.int64).astype(np.uint64)


def _grow(index, rng, free):
    """A tree with shared prefixes, a split node and one unready leaf."""
    base = _hashes(rng, 6)
    seqs = [base, np.concatenate([base[:4], _hashes(rng, 3)]), np.concatenate([base[:2], _hashes(rng, 5)]),
            _hashes(rng, 4)]
    for s in seqs:
        m = index.match_prefix(s, len(s), False)
        need = len(s) - m.num_matched_blocks
        blocks = np.asarray([free.pop() for _ in range(need)], dtype=np.int64)
        index.insert(blocks, s, len(s), True, m)
    pending = np.concatenate([seqs[3], _hashes(rng, 2)])
    blocks = np.asarray([free.pop() for _ in range(2)], dtype=np.int64)
    index.insert(blocks, pending, len(pending), False, None)
    return seqs, pending


@pytest.mark.parametrize("native", [True, False])
def test_index_image_round_trips_and_skips_unready_nodes(native):
    make = (lambda: C.RadixIndex(4, 64, "lru", 0.0, 2)) if native else (lambda: RadixTreeIndex(4, 64, "lru", 0.0, 2))
    rng = np.random.default_rng(3)
    a = make()
    seqs, pending = _grow(a, rng, list(range(63, -1, -1)))
    image = a.export_ready()
    parents, sizes, hashes, blocks = image
    assert int(sizes.sum()) == len(hashes) == len(blocks) == a.total_ready_blocks()
    assert (parents < np.arange(len(parents))).all()
    b = make()
    assert b.import_snapshot(*image) == a.total_ready_blocks()
    for s in seqs:
        ma, mb = a.match_prefix(s, len(s), False), b.match_prefix(s, len(s), False)
        assert mb.num_ready_matched_blocks == len(s)
        assert np.array_equal(np.asarray(ma.physical_blocks), np.asarray(mb.physical_blocks))
    assert b.match_prefix(pending, len(pending), False).num_matched_blocks == 4     # the unready tail is gone
    # the image of the rebuilt tree is the image it was built from
    for x, y in zip(image, b.export_ready()):
        assert np.array_equal(x, y)


def test_native_and_python_index_write_the_same_image():
    rng1, rng2 = np.random.default_rng(5), np.random.default_rng(5)
    a, b = C.RadixIndex(4, 64, "lru", 0.0, 2), RadixTreeIndex(4, 64, "lru", 0.0, 2)
    _grow(a, rng1, list(range(63, -1, -1)))
    _grow(b, rng2, list(range(63, -1, -1)))
    for x, y in zip(a.export_ready(), b.export_ready()):
        assert np.array_equal(x, y)


@pytest.mark.parametrize("native", [True, False])
def test_malformed_images_are_rejected_and_leave_the_index_empty(native):
    make = (lambda: C.RadixIndex(4, 16, "lru", 0.0, 2)) if native else (lambda: RadixTreeIndex(4, 16, "lru", 0.0, 2))
    h = np.arange(1, 5, dtype=np.uint64)
    good = (np.asarray([-1, 0], np.int32), np.asarray([2, 2], np.int64), h, np.asarray([0, 1, 2, 3], np.int64))
    bad = [
        (np.asarray([0, -1], np.int32),) + good[1:],                                  # parent after child
        (good[0], np.asarray([2, 3], np.int64)) + good[2:],                           # sizes do not cover
        good[:3] + (np.asarray([0, 1, 2, 99], np.int64),),                            # block out of range
        good[:3] + (np.asarray([0, 1, 1, 3], np.int64),),                             # block twice
        (np.asarray([-1, -1], np.int32), good[1], np.asarray([1, 2, 1, 2], np.uint64), good[3]),  # same path twice
    ]
    for image in bad:
        t = make()
        with pytest.raises((ValueError, RuntimeError)):
            t.import_snapshot(*image)
        assert t.is_empty() and t.total_cached_blocks() == 0
    t = make()
    assert t.import_snapshot(*good) == 4
    with pytest.raises((ValueError, RuntimeError)):
        t.import_snapshot(*good)                                                       # not empty


@pytest.mark.parametrize("native", [True, False])
def test_pool_reserve_takes_exactly_the_named_blocks(native):
    p = Mempool(8, native=native)
    p.reserve_blocks(np.asarray([1, 5, 6]))
    assert p.num_free_blocks == 5
    got = np.sort(p.allocate_blocks(5))
    assert got.tolist() == [0, 2, 3, 4, 7]
    p.recycle_blocks(np.asarray([5]))
    with pytest.raises((RuntimeError, IndexError)):
        p.reserve_blocks(np.asarray([5, 6]))          # 6 is in use: nothing changes
    assert p.num_free_blocks == 1
    with pytest.raises((RuntimeError, IndexError)):
        p.reserve_blocks(np.asarray([9]))
    p.reserve_blocks(np.asarray([5]))
    assert p.num_free_blocks == 0


SHAPE = KVShape("w", 3, 2, 32, tokens_per_block=4)


def _put(mgr, kv, tok, src):
    T = SHAPE.tokens_per_block
    tid = mgr.put_async(tok, slots(src, T))
    assert mgr.wait(tid, completely=True)[tid].status.value == "success"
    return chunks(kv, "vllm", SHAPE, src)


@pytest.mark.parametrize("compress", [False, True])
def test_second_manager_serves_the_first_ones_ssd_blocks(tmp_path, compress):
    T = SHAPE.tokens_per_block
    kw = dict(num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=128, ssd_cache_dir=str(tmp_path), ssd_persist=True,
              enable_compression=compress)
    rng = np.random.default_rng(0)
    tok_a = rng.integers(0, 1000, size=9 * T, dtype=np.int64)
    tok_b = np.concatenate([tok_a[:4 * T], rng.integers(0, 1000, size=6 * T, dtype=np.int64)])
    mgr, (kv,) = start(SHAPE, "vllm", **kw)
    try:
        want_a = _put(mgr, kv, tok_a, np.arange(0, 9))
        want_b = _put(mgr, kv, tok_b, np.concatenate([np.arange(0, 4), np.arange(20, 26)]))
    finally:
        mgr.shutdown()
    names = set(os.listdir(tmp_path))
    assert {"flexkv_ssd_cache.index.npz", "flexkv_ssd_cache.sizes.npy", "flexkv_ssd_cache_0_0.bin"} <= names

    mgr, (kv,) = start(SHAPE, "vllm", **kw)
    try:
        eng = mgr.kv_task_engine.cache_engine
        assert eng.ssd_blocks_restored == 15                       # 9 + 6 new blocks of the second sequence
        assert eng.ssd_cache_engine.mempool.num_used_blocks == 15
        assert "flexkv_ssd_cache.index.npz" not in os.listdir(tmp_path)       # consumed by the mount
        for t in kv:
            t.zero_()
        for tok, want, n in ((tok_a, want_a, 9), (tok_b, want_b, 10)):
            dst = rng.permutation(64)[:n]
            tid = mgr.get_async(tok, slots(dst, T))
            r = mgr.wait(tid)[tid]
            assert r.status.value == "success" and r.return_mask.sum() == n * T
            assert torch.equal(chunks(kv, "vllm", SHAPE, dst), want)
        # the mounted tier keeps working: new blocks do not land on restored ones
        tok_c = rng.integers(2000, 3000, size=5 * T, dtype=np.int64)
        want_c = _put(mgr, kv, tok_c, np.arange(40, 45))
        mgr._clear_cpu_cache()
        for t in kv:
            t.zero_()
        for tok, want, n in ((tok_a, want_a, 9), (tok_c, want_c, 5)):
            dst = rng.permutation(64)[:n]
            tid = mgr.get_async(tok, slots(dst, T))
            r = mgr.wait(tid)[tid]
            assert r.status.value == "success" and r.return_mask.sum() == n * T
            assert torch.equal(chunks(kv, "vllm", SHAPE, dst), want)
    finally:
        mgr.shutdown()


def test_unsafe_images_give_a_cold_start(tmp_path):
    T = SHAPE.tokens_per_block
    kw = dict(num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=128, ssd_cache_dir=str(tmp_path), ssd_persist=True)
    tok = np.arange(6 * T, dtype=np.int64)

    def run(put, **over):
        mgr, (kv,) = start(SHAPE, "vllm", **dict(kw, **over))
        try:
            restored = mgr.kv_task_engine.cache_engine.ssd_blocks_restored
            if put:
                _put(mgr, kv, tok, np.arange(6))
            return restored
        finally:
            mgr.shutdown()

    assert run(True) == 0
    assert run(False) == 6                                   # clean restart: mounted, saved again at shutdown
    assert run(False, num_ssd_blocks=256) == 0               # another geometry: ignored (and consumed)
    assert run(True) == 0                                    # the mismatching run saved an empty index
    path = persist.index_path(type("c", (), {"ssd_cache_dir": str(tmp_path)})())
    with open(path, "r+b") as f:                             # damaged file
        f.seek(8)
        f.write(b"\0" * 64)
    assert run(True) == 0
    # a mount without a clean shutdown after it: the image is gone, the next start is cold
    from flexkv_b200 import CacheConfig
    from flexkv_b200.cache.cache_engine import GlobalCacheEngine
    from flexkv_b200.models import make_model_config
    cc = CacheConfig(tokens_per_block=T, **kw)
    mc = make_model_config(SHAPE)
    first = GlobalCacheEngine(cc, mc)
    assert first.ssd_blocks_restored == 6
    second = GlobalCacheEngine(cc, mc)                       # "crash": first never shut down
    assert second.ssd_blocks_restored == 0


def test_checkpoint_survives_a_crash_and_is_withdrawn_when_blocks_are_about_to_be_rewritten(tmp_path, monkeypatch):
    T = SHAPE.tokens_per_block
    kw = dict(num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=16, ssd_cache_dir=str(tmp_path), ssd_persist=True)
    index_file = tmp_path / "flexkv_ssd_cache.index.npz"
    tok = np.arange(6 * T, dtype=np.int64) + 50
    mgr, (kv,) = start(SHAPE, "vllm", **kw)
    want = _put(mgr, kv, tok, np.arange(6))
    assert mgr.checkpoint_ssd_index() and index_file.exists()
    # "crash": the process state is dropped without a shutdown (threads are stopped, nothing is saved)
    monkeypatch.setenv("FLEXKV_KEEP_SSD_FILES", "1")
    mgr.kv_task_engine.cache_engine._index_saved = True           # what a killed process would not have done:
    mgr.transfer_manager.storage._ssd_persist = False             # neither the index nor the size table is rewritten
    mgr.shutdown()
    assert index_file.exists()
    mgr, (kv,) = start(SHAPE, "vllm", **kw)
    try:
        assert mgr.kv_task_engine.cache_engine.ssd_blocks_restored == 6
        for t in kv:
            t.zero_()
        dst = np.arange(10, 16)
        tid = mgr.get_async(tok, slots(dst, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        assert torch.equal(chunks(kv, "vllm", SHAPE, dst), want)
        # a new checkpoint, then the 16-block tier has to evict to take 12 more blocks: the image goes
        assert mgr.checkpoint_ssd_index() and index_file.exists()
        _put(mgr, kv, np.arange(12 * T, dtype=np.int64) + 5000, np.arange(20, 32))
        assert not index_file.exists()
    finally:
        mgr.shutdown()
    assert index_file.exists()                                     # the clean shutdown saved the current state
