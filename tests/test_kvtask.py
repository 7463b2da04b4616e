"""Task layer with a scripted fake data plane: lifecycle, wait semantics, batch
merge, cancel rollback, failure propagation over one and several handles
(reference: tests/test_kvtask_lifecycle.py, test_cancel_task_rollback.py,
test_transfer_failure_propagation.py, test_batch_kvtask.py)."""
import numpy as np
import pytest
import torch

from flexkv_b200.common.config import CacheConfig, ModelConfig
from flexkv_b200.common.request import KVResponseStatus as S
from flexkv_b200.common.transfer import CompletedOp, TransferType
from flexkv_b200.kvtask import KVTaskEngine, TaskStatus

T = 4


class FakeHandle:
    """Records submitted graphs; the test decides when and how each op finishes."""

    def __init__(self):
        self.graphs = []
        self.out = []

    def start(self): pass
    def is_ready(self): return True
    def shutdown(self): pass

    def submit_batch(self, graphs):
        self.graphs.extend(graphs)

    def wait(self, timeout=None):
        out, self.out = self.out, []
        return out

    def finish_op(self, graph, op, ok=True):
        graph.mark_completed(op.op_id, ok)
        self.out.append(CompletedOp(graph.graph_id, op.op_id, ok))

    def run(self, graph, fail_type=None, stop_after=None):
        """Executes the graph in dependency order; an op of `fail_type` fails and the graph is abandoned."""
        n = 0
        while True:
            ready = graph.take_ready_ops()
            if not ready:
                break
            for op in ready:
                if fail_type is not None and op.transfer_type == fail_type:
                    self.finish_op(graph, op, False)
                    self.out.append(CompletedOp.graph_done(graph.graph_id, success=False))
                    return
                self.finish_op(graph, op, True)
                n += 1
                if stop_after is not None and n >= stop_after:
                    return
        self.out.append(CompletedOp.graph_done(graph.graph_id, success=True))


def engine(tmp_path=None, handles=1, num_cpu=32, ssd=False):
    m = ModelConfig(num_layers=2, num_kv_heads=2, head_size=8, dtype=torch.bfloat16)
    c = CacheConfig(tokens_per_block=T, num_cpu_blocks=num_cpu, enable_ssd=ssd, num_ssd_blocks=64,
                    ssd_cache_dir=str(tmp_path) if tmp_path else None)
    hs = [FakeHandle() for _ in range(handles)]
    return KVTaskEngine(m, c, transfer_handles=hs), hs


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


TOK = np.arange(20, dtype=np.int64)


def test_put_get_lifecycle():
    e, (h,) = engine()
    tid, mask = e.put_async(TOK, slots(range(5)))
    assert mask.sum() == 20 and e.tasks[tid].status == TaskStatus.RUNNING and len(h.graphs) == 1
    assert e.try_wait([tid]) == {}                                      # not finished: omitted
    assert e.wait([tid], timeout=0.05)[tid].status == S.TIMEOUT
    h.run(h.graphs[0])
    e._update_tasks(timeout=0)
    done = e.tasks[tid]                                                 # finished, answer not fetched yet:
    assert done.graph is None and done.token_ids is None and done.slot_mapping is None     # the heavy parts are gone
    assert done.return_mask.sum() == 20
    r = e.wait([tid])[tid]
    assert r.status == S.SUCCESS and r.return_mask.sum() == 20
    assert e.wait([tid])[tid].status == S.NOTFOUND                      # released once returned
    # match-then-launch get
    gid, gmask = e.get_match(TOK)
    assert gmask.sum() == 20 and e.tasks[gid].status == TaskStatus.UNREADY
    assert e.wait([gid])[gid].status == S.UNREADY
    e.launch_tasks([gid], [slots(range(10, 15))])
    g = h.graphs[-1]
    assert list(g.ops()[0].dst_block_ids) == [10, 11, 12, 13, 14]
    h.run(g)
    assert e.try_wait([gid])[gid].status == S.SUCCESS
    assert e.wait([12345])[12345].status == S.NOTFOUND


def test_zero_hit_get_completes_immediately_and_cancel_is_harmless():
    e, (h,) = engine()
    gid, mask = e.get_match(TOK)
    assert mask.sum() == 0 and e.wait([gid])[gid].status == S.SUCCESS and not h.graphs
    e.cancel_tasks([gid])


def test_put_success_is_visible_after_end_op_before_disk_write(tmp_path):
    e, (h,) = engine(tmp_path, ssd=True)
    tid, _ = e.put_async(TOK, slots(range(5)))
    g = h.graphs[0]
    h.run(g, stop_after=1)                                              # D2H done, H2DISK not yet
    assert e.wait([tid], timeout=0.05, completely=True)[tid].status == S.TIMEOUT
    assert e.wait([tid], timeout=0.05)[tid].status == S.SUCCESS         # end op finished
    # host copy is already usable, SSD copy not yet
    assert e.cache_engine.cpu_cache_engine.match(_seq()).num_ready_matched_blocks == 5
    assert e.cache_engine.ssd_cache_engine.match(_seq()).num_ready_matched_blocks == 0
    h.run(g)
    assert e.wait([tid], completely=True)[tid].status == S.SUCCESS
    assert e.cache_engine.ssd_cache_engine.match(_seq()).num_ready_matched_blocks == 5


def _seq():
    from flexkv_b200.common.block import SequenceMeta
    return SequenceMeta(TOK, T)


def test_failed_op_gives_failed_not_timeout_and_rolls_back(tmp_path):
    e, (h,) = engine(tmp_path, ssd=True)
    tid, _ = e.put_async(TOK, slots(range(5)))
    h.run(h.graphs[0], fail_type=TransferType.D2H)
    assert e.wait([tid], timeout=1.0)[tid].status == S.FAILED
    cpu, ssd = e.cache_engine.cpu_cache_engine, e.cache_engine.ssd_cache_engine
    assert cpu.mempool.num_used_blocks == 0 and ssd.mempool.num_used_blocks == 0
    assert cpu.match(_seq()).num_matched_blocks == 0
    # disk write fails after the host copy succeeded: host keeps the data, SSD rolls back
    tid, _ = e.put_async(TOK, slots(range(5)))
    h.run(h.graphs[-1], fail_type=TransferType.H2DISK)
    assert e.wait([tid], timeout=1.0, completely=True)[tid].status == S.FAILED
    assert cpu.match(_seq()).num_ready_matched_blocks == 5 and ssd.mempool.num_used_blocks == 0
    # failed get reports the GPU blocks that must be recomputed
    gid, _ = e.get_match(TOK)
    e.launch_tasks([gid], [slots(range(30, 35))])
    h.run(h.graphs[-1], fail_type=TransferType.H2D)
    e._update_tasks()
    assert list(e.get_failed_gpu_blocks(gid)) == [30, 31, 32, 33, 34]
    assert e.wait([gid])[gid].status == S.FAILED
    assert cpu.index.node_lock_cnt(cpu.match(_seq()).last_node) == 0     # locks released


def test_task_waits_for_every_handle():
    e, (h1, h2) = engine(handles=2)
    tid, _ = e.put_async(TOK, slots(range(5)))
    g1 = h1.graphs[0]
    # both handles execute the same graph object in this fake; drive completions by hand
    op = g1.take_ready_ops()[0]
    g1.mark_completed(op.op_id, True)
    h1.out += [CompletedOp(g1.graph_id, op.op_id, True), CompletedOp.graph_done(g1.graph_id, True)]
    e._update_tasks()
    assert e.tasks[tid].status == TaskStatus.RUNNING                     # second handle still out
    h2.out += [CompletedOp(g1.graph_id, op.op_id, True), CompletedOp.graph_done(g1.graph_id, False)]
    assert e.wait([tid], timeout=1.0, completely=True)[tid].status == S.FAILED   # any failed handle fails the task


def test_cancel_unlaunched_task_rolls_back():
    e, (h,) = engine()
    pid, mask = e.put_match(TOK)
    cpu = e.cache_engine.cpu_cache_engine
    assert mask.sum() == 20 and cpu.mempool.num_used_blocks == 5
    e.cancel_tasks(pid)
    assert cpu.mempool.num_used_blocks == 0 and cpu.index.is_empty()
    assert e.wait([pid])[pid].status == S.CANCELLED
    # a running task cannot be cancelled
    tid, _ = e.put_async(TOK, slots(range(5)))
    e.cancel_tasks(tid)
    assert e.tasks[tid].status == TaskStatus.RUNNING
    h.run(h.graphs[-1])
    assert e.wait([tid])[tid].status == S.SUCCESS


def test_batch_launch_merges_and_reports_per_member_masks():
    e, (h,) = engine(num_cpu=64)
    toks = [np.arange(100 * i, 100 * i + 4 * n, dtype=np.int64) for i, n in enumerate((2, 3, 4))]
    ids = [e.put_match(t)[0] for t in toks]
    out = e.launch_tasks(ids, [slots(range(10 * i, 10 * i + n)) for i, n in enumerate((2, 3, 4))], as_batch=True)
    assert len(out) == 1 and len(h.graphs) == 1
    op = h.graphs[0].ops()[0]
    assert op.transfer_type == TransferType.D2H and list(op.src_block_ids) == [0, 1, 10, 11, 12, 20, 21, 22, 23]
    h.run(h.graphs[0])
    r = e.wait(out, completely=True)[out[0]]
    assert r.status == S.SUCCESS and [int(m.sum()) for m in r.return_mask] == [8, 12, 16]
    assert int(r.get_mask(1).sum()) == 12
    # member callbacks ran: everything is ready on the host tier
    for t in toks:
        assert e.get_match(t)[1].sum() == len(t)
    # a failing batch fails and rolls back every member
    toks2 = [np.arange(5000 + 100 * i, 5000 + 100 * i + 8, dtype=np.int64) for i in range(2)]
    ids = [e.put_match(t)[0] for t in toks2]
    used = e.cache_engine.cpu_cache_engine.mempool.num_used_blocks
    out = e.launch_tasks(ids, [slots([40, 41]), slots([42, 43])], as_batch=True)
    h.run(h.graphs[-1], fail_type=TransferType.D2H)
    assert e.wait(out, timeout=1.0)[out[0]].status == S.FAILED
    assert e.cache_engine.cpu_cache_engine.mempool.num_used_blocks == used - 4


def test_reset_cache_neuters_inflight_callbacks():
    e, (h,) = engine()
    tid, _ = e.put_async(TOK, slots(range(5)))
    pid, _ = e.put_match(np.arange(500, 520, dtype=np.int64))
    e.reset_cache()
    cpu = e.cache_engine.cpu_cache_engine
    assert cpu.index.is_empty() and cpu.mempool.num_used_blocks == 0
    assert e.wait([pid])[pid].status == S.CANCELLED
    h.run(h.graphs[0])                                                   # the in-flight copy lands afterwards
    assert e.wait([tid], completely=True)[tid].status == S.SUCCESS
    assert cpu.index.is_empty() and cpu.mempool.num_used_blocks == 0     # and did not touch the new index
    assert e.get_match(TOK)[1].sum() == 0


def test_ops_of_several_handles_join_before_their_callback_and_block_results_are_anded():
    """Two transfer handles (two nodes of one group): an op's callback runs after BOTH reported it, per-block
    results are combined with AND, and a missing or mis-sized list fails every block
    (reference: tests/test_kvtask_lifecycle.py:223-285)."""
    from flexkv_b200.common.transfer import CompletedOp
    from flexkv_b200.kvtask import KVTaskEngine

    class Handle:
        def __init__(self):
            self.out = []

        def wait(self, timeout=None):
            o, self.out = self.out, []
            return o

    eng = KVTaskEngine.__new__(KVTaskEngine)
    import threading
    eng._lock = threading.RLock()
    eng._op_reports = {}
    h0, h1 = Handle(), Handle()
    eng.transfer_handles = [h0, h1]
    seen = []
    eng._on_completed = seen.append
    h0.out = [CompletedOp(41, 73, True, block_results=(True, True, False), gpu_ms=1.0, num_bytes=10)]
    eng._update_tasks(0)
    assert seen == []                                         # one node is not the whole group
    h1.out = [CompletedOp(41, 73, True, block_results=(True, False, True), gpu_ms=2.0, num_bytes=5)]
    eng._update_tasks(0)
    assert len(seen) == 1 and seen[0].block_results == (True, False, False) and seen[0].success
    assert seen[0].gpu_ms == 2.0 and seen[0].num_bytes == 15 and eng._op_reports == {}
    for second in (None, (True, True)):
        seen.clear()
        h0.out = [CompletedOp(43, 76, True, block_results=(True, True, True))]
        h1.out = [CompletedOp(43, 76, True, block_results=second)]
        eng._update_tasks(0)
        assert [c.block_results for c in seen] == [(False, False, False)]
    seen.clear()
    h0.out = [CompletedOp(44, 1, True)]
    h1.out = [CompletedOp(44, 1, False), CompletedOp.graph_done(44, success=False)]
    eng._update_tasks(0)
    assert [(c.op_id, c.success, c.block_results) for c in seen] == [(1, False, None), (-1, False, None)]
