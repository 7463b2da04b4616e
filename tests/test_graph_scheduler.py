"""Native transfer-graph scheduler against the Python specification (TransferOpGraph + the
scheduler loop of engine_spec.py): random DAGs with instant (virtual / empty) ops, scripted op
failures, fan-out joins, requeue; and the two engines end to end with scripted workers."""
import random
import threading

import numpy as np
import pytest

from flexkv_b200 import _native
from flexkv_b200.common.transfer import TransferOp, TransferOpGraph, TransferType, WorkerKey
from flexkv_b200.transfer.engine import TransferEngine
from flexkv_b200.transfer.engine_spec import TransferEngineSpec
from flexkv_b200.transfer.workers import OpOutcome, TransferWorker

C = _native.C
IDS = np.arange(4, dtype=np.int64)


def random_graph(rng: random.Random, n: int):
    g = TransferOpGraph()
    ops = []
    for i in range(n):
        if rng.random() < 0.2:
            oid = g.add_virtual_op([])
            ops.append(g.get_op(oid))
        else:
            empty = rng.random() < 0.1
            op = TransferOp(g.graph_id, TransferType.H2DISK, IDS[:0] if empty else IDS, IDS[:0] if empty else IDS)
            g.add_transfer_op(op)
            ops.append(op)
        for j in range(i):
            if rng.random() < 0.25:
                g.add_dependency(ops[i].op_id, ops[j].op_id)
    return g, ops


def is_instant(op):
    return op.transfer_type == TransferType.VIRTUAL or op.valid_block_num == 0


def run_spec(g, fail):
    """The specification's walk: take ready ops, instant ones complete at once, the running op with the
    smallest id finishes next; a failed graph takes nothing more and ends when nothing runs."""
    log, running = [], []
    def dispatch():
        progress = not g.failed
        while progress:
            progress = False
            for op in g.take_ready_ops():
                if is_instant(op):
                    g.mark_completed(op.op_id, True)
                    log.append(("done", op.op_id, True))
                    progress = True
                else:
                    running.append(op.op_id)
                    log.append(("run", op.op_id))
    dispatch()
    while running:
        running.sort()
        oid = running.pop(0)
        ok = oid not in fail
        g.mark_completed(oid, ok)
        log.append(("done", oid, ok))
        dispatch()
    log.append(("graph", not g.failed))
    return log


def run_native(g, ops, fail):
    s = C.GraphScheduler()
    flags = [C.SCHED_OP_INSTANT if is_instant(op) else 0 for op in ops]
    edges = [(op.op_id, p) for op in ops for p in op.predecessors]
    log, running = [], []
    ready = s.submit(g.graph_id, [op.op_id for op in ops], flags, edges)
    def drain():
        for gid, oid, ok, ms, nb in s.wait(0.0):
            log.append(("graph", ok) if oid < 0 else ("done", oid, ok))
    def take(ready):
        # completion records of instant ops precede the hand-out of what they released
        drain()
        for oid in ready:
            running.append(oid)
            log.append(("run", oid))
    take(ready)
    while running:
        running.sort()
        oid = running.pop(0)
        acc, fin, ok, ms, nb, gdone, gfail, ready = s.op_done(g.graph_id, oid, oid not in fail, 1.0, 8)
        assert acc and fin and ok == (oid not in fail)
        take(ready)
    drain()
    assert not s.has_graph(g.graph_id)
    return log


def normalise(log):
    """Both walks agree on WHICH ops run and finish and how; the interleaving of the completion records of
    instant ops with hand-outs inside one release step is not part of the contract."""
    return (sorted(e for e in log if e[0] == "run"), sorted(e for e in log if e[0] == "done"),
            [e for e in log if e[0] == "graph"])


@pytest.mark.parametrize("seed", range(40))
def test_random_graphs_match_the_specification(seed):
    rng = random.Random(seed)
    n = rng.randint(1, 14)
    state = rng.getstate()
    g1, ops1 = random_graph(rng, n)
    rng.setstate(state)
    g2, ops2 = random_graph(rng, n)
    real = [i for i, op in enumerate(ops1) if not is_instant(op)]
    bad_idx = set(rng.sample(real, k=min(len(real), rng.choice([0, 0, 1, 2]))))
    a = run_spec(g1, {ops1[i].op_id for i in bad_idx})
    b = run_native(g2, ops2, {ops2[i].op_id for i in bad_idx})
    # op ids differ between the two graphs (a global counter): compare by position
    pos1 = {op.op_id: i for i, op in enumerate(ops1)}
    pos2 = {op.op_id: i for i, op in enumerate(ops2)}
    ra = normalise([(e[0], pos1[e[1]], *e[2:]) if e[0] != "graph" else e for e in a])
    rb = normalise([(e[0], pos2[e[1]], *e[2:]) if e[0] != "graph" else e for e in b])
    assert ra == rb


def test_fanout_join_and_requeue():
    s = C.GraphScheduler()
    assert s.submit(7, [1, 2], [0, 0], [(2, 1)]) == [1]
    s.set_fanout(7, 1, 3)
    assert s.op_done(7, 1, True, 2.0, 10)[:2] == (True, False)
    assert s.op_done(7, 1, False, 5.0, 10)[:2] == (True, False)          # one stage failed
    acc, fin, ok, ms, nb, gdone, gfail, ready = s.op_done(7, 1, True, 1.0, 10)
    assert (fin, ok, ms, nb, gdone, gfail, ready) == (True, False, 5.0, 30, True, True, [])
    assert s.op_done(7, 1, True, 0.0, 0)[0] is False                      # the graph is gone: report ignored
    recs = s.wait(0.0)
    assert [(r[1], r[2]) for r in recs] == [(1, False), (-1, False)]
    # requeue: an op handed out but not started goes back and is handed out again
    assert s.submit(8, [5], [0], []) == [5]
    assert s.requeue(8, 5) and s.take_ready(8) == [5] and s.take_ready(8) == []
    assert s.op_done(8, 5, True, 0.0, 0)[5] is True
    assert s.stats()["graphs"] == 2 and s.stats()["failed_graphs"] == 1
    with pytest.raises(ValueError):
        s.submit(9, [1, 1], [0, 0], [])
    with pytest.raises(ValueError):
        s.submit(9, [1], [0], [(1, 1)])


def test_wait_blocks_without_the_gil_until_a_completion_arrives():
    s = C.GraphScheduler()
    s.submit(1, [1], [0], [])
    got = []
    th = threading.Thread(target=lambda: got.extend(s.wait(5.0)))
    th.start()
    assert s.wait(0.0) == [] and th.is_alive()
    s.op_done(1, 1, True, 0.5, 4)
    th.join(5)
    assert [(r[0], r[1], r[2]) for r in got] == [(1, 1, True), (1, -1, True)]
    assert s.wait(0.01) == []


class ScriptedWorker(TransferWorker):
    name = "scripted"

    def __init__(self, fail_ops):
        super().__init__()
        self.fail_ops = fail_ops
        self.seen = []

    def execute(self, op):
        self.seen.append(op.op_id)
        return OpOutcome(op.op_id not in self.fail_ops, gpu_ms=0.25, num_bytes=64)


class FakeModel:
    local_pp_stages = 1


@pytest.mark.parametrize("engine_cls", [TransferEngine, TransferEngineSpec])
@pytest.mark.parametrize("fail_second", [False, True])
def test_both_engines_report_the_same_completions(engine_cls, fail_second):
    g = TransferOpGraph()
    a = TransferOp(g.graph_id, TransferType.H2DISK, IDS, IDS)
    b = TransferOp(g.graph_id, TransferType.H2DISK, IDS, IDS)
    c = TransferOp(g.graph_id, TransferType.H2DISK, IDS, IDS)
    for op in (a, b, c):
        g.add_transfer_op(op)
    g.add_dependency(b.op_id, a.op_id)
    g.add_dependency(c.op_id, b.op_id)
    v = g.add_virtual_op([a.op_id])
    w = ScriptedWorker({b.op_id} if fail_second else set())
    eng = engine_cls(None, FakeModel(), None, workers={(WorkerKey(0, 0), TransferType.H2DISK): w})
    eng.start()
    try:
        eng.submit(g)
        recs = []
        for _ in range(200):
            recs += eng.wait(0.05)
            if any(r.is_graph_done() if hasattr(r, "is_graph_done") else r.op_id < 0 for r in recs):
                break
    finally:
        eng.shutdown()
    ops = {(r.op_id, r.success) for r in recs if r.op_id >= 0}
    done = [r for r in recs if r.op_id < 0]
    if fail_second:
        assert ops == {(a.op_id, True), (v, True), (b.op_id, False)} and w.seen == [a.op_id, b.op_id]
        assert len(done) == 1 and not done[0].success
    else:
        assert ops == {(a.op_id, True), (v, True), (b.op_id, True), (c.op_id, True)}
        assert len(done) == 1 and done[0].success
