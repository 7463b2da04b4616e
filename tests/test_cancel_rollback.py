"""Cancel / abort of plans and what they leave behind in the tiers (reference scenarios:
tests/test_cancel_task_rollback.py): a rollback removes only what is safe to remove, a plan handle runs one path
once, aborted plans give every block back on every tier, and raced plans leave no lock behind."""
import numpy as np
import pytest
import torch

from flexkv_b200.cache.cache_engine import CacheEngine, GlobalCacheEngine, TransferPlanHandle
from flexkv_b200.common.block import SequenceMeta
from flexkv_b200.common.config import CacheConfig, ModelConfig
from flexkv_b200.common.transfer import DeviceType

T = 4


def seq(n, seed):
    rng = np.random.default_rng(seed)
    return SequenceMeta(rng.integers(0, 1 << 30, size=n * T, dtype=np.int64), T)


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def tier(accel):
    return CacheEngine(DeviceType.CPU, 16, T, accel=accel)


def make_global(tmp_path=None, ssd=0):
    m = ModelConfig(num_layers=2, num_kv_heads=2, head_size=8, dtype=torch.bfloat16)
    c = CacheConfig(tokens_per_block=T, num_cpu_blocks=16, enable_ssd=ssd > 0, num_ssd_blocks=max(ssd, 1),
                    ssd_cache_dir=str(tmp_path) if tmp_path else None)
    return GlobalCacheEngine(c, m)


def run_ops(graph, cbs, g):
    done = set()
    while len(done) < graph.num_ops:
        for op in graph.take_ready_ops():
            graph.mark_completed(op.op_id, True)
            if op.op_id in cbs:
                g.run_op_callback(cbs[op.op_id])
            done.add(op.op_id)


def locks_left(engine):
    idx = engine.index
    if hasattr(idx, "total_locked_nodes"):
        return idx.total_locked_nodes()
    return None


@pytest.mark.parametrize("accel", [True, False])
def test_rollback_removes_an_unready_unlocked_leaf_and_nothing_else(accel):
    e = tier(accel)
    s = seq(3, 1)
    node = e.insert(s, e.take(3), is_ready=False)
    assert e.mempool.num_used_blocks == 3
    assert e.rollback_unready_insert(node) == 3 and e.mempool.num_used_blocks == 0
    assert e.match(s).num_matched_blocks == 0
    # ready node: its blocks hold data somebody may be reading
    node = e.insert(s, e.take(3), is_ready=True)
    assert e.rollback_unready_insert(node) == 0 and e.mempool.num_used_blocks == 3
    # locked node: a plan still references it
    s2 = seq(2, 2)
    n2 = e.insert(s2, e.take(2), is_ready=False)
    e.lock_node(n2)
    assert e.rollback_unready_insert(n2) == 0 and e.mempool.num_used_blocks == 5
    e.unlock(n2)
    # a node that gained a child: another request extended it in the meantime
    longer = SequenceMeta(np.concatenate([s2.token_ids, seq(1, 3).token_ids]), T)
    e.insert(longer, e.take(1), is_ready=False, match_result=e.match(longer))
    assert e.rollback_unready_insert(n2) == 0 and e.mempool.num_used_blocks == 6
    assert e.rollback_unready_insert(None) == 0


def test_a_plan_handle_runs_one_path_once():
    calls = []
    h = TransferPlanHandle(lambda: calls.append("complete"), lambda: calls.append("abort"))
    h.complete(); h.complete(); h.abort()
    assert calls == ["complete"]
    calls.clear()
    h = TransferPlanHandle(lambda: calls.append("complete"), lambda: calls.append("abort"))
    h.abort(); h.complete(); h.abort()
    assert calls == ["abort"]


def test_aborted_put_gives_every_block_back_on_both_tiers(tmp_path):
    g = make_global(tmp_path, ssd=32)
    s = seq(5, 10)
    graph, mask, handle, cbs, _ = g.put(0, s.token_ids, None, slots(range(5)))
    assert mask.sum() == 5 * T
    assert g.cpu_cache_engine.mempool.num_used_blocks == 5 and g.ssd_cache_engine.mempool.num_used_blocks == 5
    handle.abort()
    for e in (g.cpu_cache_engine, g.ssd_cache_engine):
        assert e.mempool.num_used_blocks == 0 and e.match(s).num_matched_blocks == 0
    handle.abort(); handle.complete()                       # late calls change nothing
    assert g.cpu_cache_engine.mempool.num_used_blocks == 0
    # and the tiers are usable: the same put goes through afterwards
    graph, mask, handle, cbs, _ = g.put(1, s.token_ids, None, slots(range(5)))
    run_ops(graph, cbs, g)
    handle.complete()
    assert g.cpu_cache_engine.match(s).num_ready_matched_blocks == 5
    assert g.ssd_cache_engine.match(s).num_ready_matched_blocks == 5


def test_aborted_get_returns_its_staging_blocks(tmp_path):
    """A get that has to stage SSD blocks in the host pool takes host blocks at plan time; aborting gives them back."""
    g = make_global(tmp_path, ssd=32)
    s = seq(4, 20)
    graph, _, handle, cbs, _ = g.put(0, s.token_ids, None, slots(range(4)))
    run_ops(graph, cbs, g)
    handle.complete()
    g.cpu_cache_engine.index.reset(); g.cpu_cache_engine.mempool.reset()       # only the SSD tier keeps the prefix
    used0 = g.cpu_cache_engine.mempool.num_used_blocks
    graph, mask, handle, cbs, _ = g.get(1, s.token_ids, None, None)
    assert mask.sum() == 4 * T and g.cpu_cache_engine.mempool.num_used_blocks == used0 + 4
    handle.abort()
    assert g.cpu_cache_engine.mempool.num_used_blocks == used0
    assert g.cpu_cache_engine.match(s).num_matched_blocks == 0
    assert g.ssd_cache_engine.match(s).num_ready_matched_blocks == 4            # the source is untouched


def test_completed_then_cancelled_plan_releases_once():
    g = make_global()
    s = seq(3, 30)
    graph, _, handle, cbs, _ = g.put(0, s.token_ids, None, slots(range(3)))
    run_ops(graph, cbs, g)
    handle.complete()
    handle.abort()                                          # a cancel that arrives after the task finished
    cpu = g.cpu_cache_engine
    assert cpu.mempool.num_used_blocks == 3 and cpu.match(s).num_ready_matched_blocks == 3
    m = cpu.match(s)
    with pytest.raises(RuntimeError):
        cpu.index.unlock(m.last_node)                       # nothing is left locked: one more unlock is an error


def test_cancel_with_a_pending_extension_leaves_a_bounded_unlocked_hole():
    """Put B (prefix + extension) is planned while put A (prefix) is pending: B skips A's blocks. Cancelling A
    cannot remove A's node any more (B's node hangs below it), so the prefix stays unready: nobody wrote it. The
    hole is exactly A's insert and nothing stays locked once both plans are resolved."""
    g = make_global()
    cpu = g.cpu_cache_engine
    a = seq(4, 61)
    b = SequenceMeta(np.concatenate([a.token_ids, seq(2, 62).token_ids]), T)
    graph_a, mask_a, handle_a, cbs_a, _ = g.put(1, a.token_ids, None, slots(range(4)))
    graph_b, mask_b, handle_b, cbs_b, _ = g.put(2, b.token_ids, None, slots(range(6)))
    assert mask_a.sum() == 4 * T and mask_b.sum() == 2 * T and not mask_b[:4 * T].any()
    handle_a.abort()
    run_ops(graph_b, cbs_b, g)
    handle_b.complete()
    assert cpu.index.total_cached_blocks() - cpu.index.total_ready_blocks() == 4          # A's insert, no more
    m = cpu.match(b)
    assert m.num_matched_blocks == 6 and m.num_ready_matched_blocks == 0     # a ready match is a contiguous prefix
    assert cpu.mempool.num_used_blocks == 6
    # nothing is locked: unlocking either node once more is an error
    for s_ in (a, b):
        with pytest.raises(RuntimeError):
            cpu.index.unlock(cpu.match(s_).last_node)


def test_cancelled_get_with_a_racing_put_leaves_no_residue():
    g = make_global()
    cpu = g.cpu_cache_engine
    s = seq(4, 71)
    graph, _, handle, cbs, _ = g.put(0, s.token_ids, None, slots(range(4)))
    run_ops(graph, cbs, g)
    handle.complete()
    # a get is planned (locks the node), an extending put arrives, the get is cancelled, the put completes
    graph_g, mask_g, handle_g, _, _ = g.get(1, s.token_ids, None, None)
    assert mask_g.sum() == 4 * T
    longer = SequenceMeta(np.concatenate([s.token_ids, seq(2, 72).token_ids]), T)
    graph_p, mask_p, handle_p, cbs_p, _ = g.put(2, longer.token_ids, None, slots(range(6)))
    assert mask_p.sum() == 2 * T
    handle_g.abort()
    run_ops(graph_p, cbs_p, g)
    handle_p.complete()
    assert cpu.match(longer).num_ready_matched_blocks == 6 and cpu.mempool.num_used_blocks == 6
    assert len(cpu.index.evict(16)[0]) == 6 and cpu.index.is_empty()            # nothing was left locked
