"""Tier engine and planner: config validation, pool, take/evict, put and get
plans with host and SSD tiers, abort/rollback (reference: tests/test_cache_engine.py,
tests/test_cancel_task_rollback.py)."""
import numpy as np
import pytest
import torch

from flexkv_b200.cache.cache_engine import CacheEngine, GlobalCacheEngine
from flexkv_b200.cache.mempool import Mempool, NotEnoughSpaceError
from flexkv_b200.common.block import SequenceMeta
from flexkv_b200.common.config import CacheConfig, ModelConfig
from flexkv_b200.common.transfer import DeviceType, TransferType

T = 4


def seq(tokens):
    return SequenceMeta(np.asarray(tokens, dtype=np.int64), T)


@pytest.mark.parametrize("native", [True, False])
def test_mempool(native):
    p = Mempool(8, native=native)
    a = p.allocate_blocks(5)
    assert len(set(a.tolist())) == 5 and p.num_free_blocks == 3
    with pytest.raises(NotEnoughSpaceError):
        p.allocate_blocks(4)
    assert len(p.allocate_blocks(4, strict=False)) == 3 and p.num_free_blocks == 0
    p.recycle_blocks(a[:2])
    with pytest.raises(RuntimeError):
        p.recycle_blocks(a[:1])                      # double free
    with pytest.raises(RuntimeError):
        p.recycle_blocks(np.array([a[2], a[2]]))     # duplicate in one call
    assert p.num_free_blocks == 2                    # failed calls changed nothing
    with pytest.raises((IndexError, RuntimeError)):
        p.recycle_blocks(np.array([99]))
    p.reset()
    assert p.num_free_blocks == 8


@pytest.mark.parametrize("kw", [dict(num_total_blocks=0), dict(tokens_per_block=3), dict(evict_ratio=1.5),
                                dict(evict_start_threshold=0.0)])
def test_config_validation(kw):
    args = dict(device_type=DeviceType.CPU, num_total_blocks=8, tokens_per_block=4)
    args.update(kw)
    with pytest.raises(ValueError):
        CacheEngine(**args)


@pytest.mark.parametrize("accel", [True, False])
def test_take_evicts_lru_and_respects_threshold(accel):
    e = CacheEngine(DeviceType.CPU, 10, T, accel=accel)
    e.index.set_clock_override(1)
    s1, s2 = seq(range(16)), seq(range(100, 116))
    e.insert(s1, e.take(4), is_ready=True)
    e.index.set_clock_override(2)
    e.insert(s2, e.take(4), is_ready=True)
    assert e.mempool.num_free_blocks == 2
    got = e.take(4)                                   # needs 2 more: evicts from the older sequence's tail
    assert len(got) == 4 and e.match(s1).num_matched_blocks == 2 and e.match(s2).num_matched_blocks == 4
    with pytest.raises(NotEnoughSpaceError):
        e.take(100)
    assert len(e.take(100, strict=False)) == 6       # everything evictable goes: 10 blocks minus the 4 just taken
    # proactive eviction: above 50 % utilisation fall back under it, at least evict_ratio * total
    e2 = CacheEngine(DeviceType.CPU, 10, T, evict_ratio=0.3, evict_start_threshold=0.5, accel=accel)
    e2.insert(seq(range(24)), e2.take(6), is_ready=True)
    e2.take(1)
    assert e2.num_evicted_total >= 3 and e2.mempool.num_used_blocks <= 5


def make_global(num_cpu=16, num_ssd=0, tmp=None, **kw):
    m = ModelConfig(num_layers=2, num_kv_heads=2, head_size=8, dtype=torch.bfloat16)
    c = CacheConfig(tokens_per_block=T, num_cpu_blocks=num_cpu, enable_ssd=num_ssd > 0, num_ssd_blocks=max(num_ssd, 1),
                    ssd_cache_dir=tmp, **kw)
    return GlobalCacheEngine(c, m)


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def run_plan(graph, cbs, g, success=True):
    """Pretend the data plane executed the graph."""
    done = set()
    while len(done) < graph.num_ops:
        for op in graph.take_ready_ops():
            graph.mark_completed(op.op_id, True)
            if op.op_id in cbs:
                g.run_op_callback(cbs[op.op_id])
            done.add(op.op_id)


def test_put_then_get_plans_host_only():
    g = make_global()
    tok = np.arange(4 * 5 + 2, dtype=np.int64)
    graph, mask, handle, cbs, end = g.put(0, tok, None, np.concatenate([slots([7, 8, 9, 10, 11]), [0, 1]]))
    ops = graph.ops()
    assert [o.transfer_type for o in ops] == [TransferType.D2H]
    assert list(ops[0].src_block_ids) == [7, 8, 9, 10, 11] and len(ops[0].dst_block_ids) == 5
    assert mask.sum() == 20 and not mask[20:].any() and end == ops[0].op_id
    # in flight: matched but not ready; a get finds nothing, a second put skips everything
    assert g.get(1, tok, None, None)[1].sum() == 0
    assert g.put(2, tok, None, None)[0].num_ops == 0
    run_plan(graph, cbs, g)
    handle.complete()
    graph2, mask2, handle2, cbs2, _ = g.get(3, tok, None, None)
    op = graph2.ops()[0]
    assert op.transfer_type == TransferType.H2D and op.gpu_side == "dst" and mask2.sum() == 20
    assert list(op.src_block_ids) == list(ops[0].dst_block_ids)
    graph2.set_gpu_blocks(np.array([1, 2, 3, 4, 5]))
    assert list(op.dst_block_ids) == [1, 2, 3, 4, 5]
    handle2.complete()
    # partially computed request: only the tail is restored, indices start at the window
    tm = np.zeros_like(tok, dtype=bool)
    tm[8:] = True
    graph3, mask3, h3, _, _ = g.get(4, tok, tm, np.concatenate([slots([40, 41, 42]), [0, 0]]))
    op = graph3.ops()[0]
    assert list(op.dst_block_ids) == [40, 41, 42] and list(op.src_block_ids) == list(ops[0].dst_block_ids[2:])
    assert mask3[8:20].all() and not mask3[:8].any() and not mask3[20:].any()
    h3.complete()
    # extending put only moves the new blocks
    tok2 = np.concatenate([tok[:20], np.arange(1000, 1008)])
    graph4, mask4, h4, cbs4, _ = g.put(5, tok2, None, slots(range(20, 27)))
    op = graph4.ops()[0]
    assert list(op.src_block_ids) == [25, 26] and mask4.sum() == 8 and mask4[20:].all()
    h4.abort()                                         # never executed: blocks and node are returned
    assert g.cpu_cache_engine.mempool.num_used_blocks == 5
    assert g.cpu_cache_engine.match(SequenceMeta(tok2, T)).num_matched_blocks == 5


def test_put_mask_must_be_a_prefix_and_full_pool_gives_empty_plan():
    g = make_global(num_cpu=4)
    tok = np.arange(32, dtype=np.int64)
    tm = np.zeros(32, dtype=bool)
    tm[8:] = True
    with pytest.raises(ValueError):
        g.put(0, tok, tm, None)
    # 8 blocks never fit in a pool of 4 whose content is locked by an in-flight put
    graph, mask, handle, cbs, _ = g.put(1, tok[:16], None, None)
    assert graph.num_ops == 1
    graph2, mask2, h2, _, _ = g.put(2, np.arange(100, 132), None, None)
    assert graph2.num_ops == 0 and mask2.sum() == 0   # silently not cached
    assert g.cpu_cache_engine.mempool.num_used_blocks == 4
    handle.abort()
    assert g.cpu_cache_engine.mempool.num_used_blocks == 0


def test_ssd_tier_plans(tmp_path):
    g = make_global(num_cpu=8, num_ssd=32, tmp=str(tmp_path))
    tok = np.arange(24, dtype=np.int64)
    graph, mask, handle, cbs, end = g.put(0, tok, None, slots(range(6)))
    kinds = {o.transfer_type: o for o in graph.ops()}
    assert set(kinds) == {TransferType.D2H, TransferType.H2DISK}
    assert kinds[TransferType.H2DISK].predecessors == {kinds[TransferType.D2H].op_id}
    assert list(kinds[TransferType.H2DISK].src_block_ids) == list(kinds[TransferType.D2H].dst_block_ids)
    assert end == kinds[TransferType.D2H].op_id        # success is reported after the GPU->host copy
    run_plan(graph, cbs, g)
    handle.complete()
    g.cpu_cache_engine.reset()                          # host tier lost, SSD keeps the blocks
    graph2, mask2, h2, cbs2, end2 = g.get(1, tok, None, None)
    kinds2 = {o.transfer_type: o for o in graph2.ops()}
    assert set(kinds2) == {TransferType.DISK2H, TransferType.H2D} and mask2.sum() == 24
    assert list(kinds2[TransferType.DISK2H].src_block_ids) == list(kinds[TransferType.H2DISK].dst_block_ids)
    assert list(kinds2[TransferType.H2D].src_block_ids) == list(kinds2[TransferType.DISK2H].dst_block_ids)
    assert kinds2[TransferType.H2D].predecessors == {kinds2[TransferType.DISK2H].op_id}
    # the staged blocks entered the host index unready and become ready when the disk read lands
    s = SequenceMeta(tok, T)
    assert g.cpu_cache_engine.match(s).num_matched_blocks == 6
    assert g.cpu_cache_engine.match(s).num_ready_matched_blocks == 0
    graph2.set_gpu_blocks(np.arange(6))
    run_plan(graph2, cbs2, g)
    h2.complete()
    assert g.cpu_cache_engine.match(s).num_ready_matched_blocks == 6
    # prefetch: SSD -> host only
    g.cpu_cache_engine.reset()
    graph3, mask3, h3, cbs3, _ = g.get(2, tok, None, None, prefetch=True)
    assert [o.transfer_type for o in graph3.ops()] == [TransferType.DISK2H] and mask3.sum() == 24
    run_plan(graph3, cbs3, g)
    h3.complete()
    assert g.cpu_cache_engine.match(s).num_ready_matched_blocks == 6
    # cpu_only ignores the SSD tier
    g.cpu_cache_engine.reset()
    assert g.get(3, tok, None, None, cpu_only=True)[0].num_ops == 0


def test_gds_get_plan_reads_disk_straight_into_the_gpu_tail(tmp_path):
    g = make_global(num_cpu=8, num_ssd=32, tmp=str(tmp_path), enable_gds=True)
    tok = np.arange(32, dtype=np.int64)
    graph, _, handle, cbs, _ = g.put(0, tok, None, slots(range(8)))
    run_plan(graph, cbs, g)
    handle.complete()
    # keep only the first 3 blocks on the host
    g.cpu_cache_engine.reset()
    gr, _, h, c, _ = g.put(1, tok[:12], None, slots(range(3)))
    run_plan(gr, c, g)
    h.complete()
    graph2, mask2, h2, _, end = g.get(2, tok, None, None)
    kinds = {o.transfer_type: o for o in graph2.ops()}
    assert set(kinds) == {TransferType.H2D, TransferType.DISK2D, TransferType.VIRTUAL} and mask2.sum() == 32
    assert not kinds[TransferType.H2D].predecessors and not kinds[TransferType.DISK2D].predecessors  # in parallel
    graph2.set_gpu_blocks(np.arange(50, 58))
    assert list(kinds[TransferType.H2D].dst_block_ids) == [50, 51, 52]
    assert list(kinds[TransferType.DISK2D].dst_block_ids) == [53, 54, 55, 56, 57]
    h2.abort()


def test_reset_and_namespace():
    g = make_global()
    tok = np.arange(16, dtype=np.int64)
    graph, _, handle, cbs, _ = g.put(0, tok, None, slots(range(4)), namespace=["a"])
    run_plan(graph, cbs, g)
    handle.complete()
    assert g.get(1, tok, None, None, namespace=["a"])[1].sum() == 16
    assert g.get(2, tok, None, None, namespace=["b"])[1].sum() == 0
    assert g.get(3, tok, None, None)[1].sum() == 0
    g.reset()
    assert g.get(4, tok, None, None, namespace=["a"])[1].sum() == 0
    assert g.cpu_cache_engine.mempool.num_used_blocks == 0
