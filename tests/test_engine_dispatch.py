"""Dispatch accounting of the transfer engine with scripted workers: which worker an op reaches, how many
executors an op waits for, and that a graph is closed exactly once whatever the workers report
(reference scenarios: tests/test_transfer_engine_atomic_eviction.py — pending-count bookkeeping, routing by
worker key, unknown routing keys, completions that arrive twice). Both engines (native scheduler and the Python
specification) must behave the same."""
import threading
import time

import numpy as np
import pytest

from flexkv_b200.common.transfer import TransferOp, TransferOpGraph, TransferOpStatus, TransferType, WorkerKey
from flexkv_b200.transfer.engine import TransferEngine
from flexkv_b200.transfer.engine_spec import TransferEngineSpec
from flexkv_b200.transfer.workers import OpOutcome, TransferWorker

IDS = np.arange(4, dtype=np.int64)
ENGINES = [TransferEngine, TransferEngineSpec]


class Recorder(TransferWorker):
    def __init__(self, name, ok=True, hold=None):
        super().__init__()
        self.name, self.ok, self.hold = name, ok, hold
        self.seen = []

    def execute(self, op):
        self.seen.append(op.op_id)
        if self.hold is not None:
            self.hold.wait(5)
        return OpOutcome(self.ok, gpu_ms=0.1, num_bytes=16)


class Model:
    def __init__(self, stages=1):
        self.local_pp_stages = stages


def drain(eng, gid, limit=5.0):
    recs, t0 = [], time.monotonic()
    while time.monotonic() - t0 < limit:
        recs += eng.wait(0.05)
        if any(r.op_id < 0 and r.graph_id == gid for r in recs):
            # nothing may follow the record that closes the graph
            time.sleep(0.05)
            recs += eng.wait(0.0)
            return recs
    raise AssertionError(f"graph {gid} never closed: {[(r.op_id, r.success) for r in recs]}")


def one_op_graph(tt, dp=0):
    g = TransferOpGraph()
    op = TransferOp(g.graph_id, tt, IDS, IDS, dp_client_id=dp)
    g.add_transfer_op(op)
    return g, op


@pytest.mark.parametrize("engine_cls", ENGINES)
def test_gpu_ops_reach_the_worker_of_their_own_client_only(engine_cls):
    w0, w1, disk = Recorder("dp0"), Recorder("dp1"), Recorder("disk")
    eng = engine_cls(None, Model(), None, workers={(WorkerKey(0, 0), TransferType.D2H): w0,
                                                    (WorkerKey(1, 0), TransferType.D2H): w1,
                                                    (WorkerKey(0, 0), TransferType.H2DISK): disk})
    eng.start()
    try:
        g, op = one_op_graph(TransferType.D2H, dp=1)
        eng.submit(g)
        recs = drain(eng, g.graph_id)
        assert w1.seen == [op.op_id] and w0.seen == []
        assert [(r.op_id, r.success) for r in recs] == [(op.op_id, True), (-1, True)]
        # tier-to-tier workers are shared: client 1's disk write goes to the one SSD worker
        g2, op2 = one_op_graph(TransferType.H2DISK, dp=1)
        eng.submit(g2)
        drain(eng, g2.graph_id)
        assert disk.seen == [op2.op_id]
    finally:
        eng.shutdown()


@pytest.mark.parametrize("engine_cls", ENGINES)
def test_an_op_nobody_can_run_fails_its_graph_instead_of_waiting(engine_cls):
    eng = engine_cls(None, Model(), None, workers={(WorkerKey(0, 0), TransferType.D2H): Recorder("dp0")})
    eng.start()
    try:
        g = TransferOpGraph()
        a = TransferOp(g.graph_id, TransferType.D2H, IDS, IDS, dp_client_id=7)      # no such client
        b = TransferOp(g.graph_id, TransferType.D2H, IDS, IDS, dp_client_id=0)
        g.add_transfer_op(a); g.add_transfer_op(b)
        g.add_dependency(b.op_id, a.op_id)
        eng.submit(g)
        recs = drain(eng, g.graph_id)
        assert (a.op_id, False) in [(r.op_id, r.success) for r in recs]
        assert [r.success for r in recs if r.op_id < 0] == [False]
        assert b.op_id not in [r.op_id for r in recs]           # the successor was never handed out
        assert a.status == TransferOpStatus.FAILED
    finally:
        eng.shutdown()


@pytest.mark.parametrize("engine_cls", ENGINES)
def test_an_op_of_several_pipeline_stages_waits_for_every_stage(engine_cls):
    gate = threading.Event()
    s0, s1, s2 = Recorder("pp0"), Recorder("pp1", hold=gate), Recorder("pp2")
    eng = engine_cls(None, Model(stages=3), None, workers={(WorkerKey(0, 0), TransferType.H2D): s0,
                                                            (WorkerKey(0, 1), TransferType.H2D): s1,
                                                            (WorkerKey(0, 2), TransferType.H2D): s2})
    eng.start()
    try:
        g, op = one_op_graph(TransferType.H2D)
        eng.submit(g)
        t0 = time.monotonic()
        while not (s0.seen and s2.seen and s1.seen) and time.monotonic() - t0 < 5:
            time.sleep(0.005)
        assert s0.seen == s1.seen == s2.seen == [op.op_id]
        time.sleep(0.05)
        assert eng.wait(0.0) == [] and op.pending_count >= 1     # two stages reported, one still holds the op
        gate.set()
        recs = drain(eng, g.graph_id)
        assert [(r.op_id, r.success) for r in recs] == [(op.op_id, True), (-1, True)]
        assert op.status == TransferOpStatus.COMPLETED
    finally:
        gate.set()
        eng.shutdown()


@pytest.mark.parametrize("engine_cls", ENGINES)
def test_a_completion_reported_twice_closes_the_graph_once(engine_cls):
    w = Recorder("dp0")
    eng = engine_cls(None, Model(), None, workers={(WorkerKey(0, 0), TransferType.D2H): w})
    eng.start()
    try:
        g, op = one_op_graph(TransferType.D2H)
        eng.submit(g)
        recs = drain(eng, g.graph_id)
        eng._on_worker_done(op, OpOutcome(True))                # a late duplicate from a confused worker
        eng._on_worker_done(op, OpOutcome(False))
        time.sleep(0.05)
        recs += eng.wait(0.0)
        assert [(r.op_id, r.success) for r in recs] == [(op.op_id, True), (-1, True)]
        assert op.status == TransferOpStatus.COMPLETED
    finally:
        eng.shutdown()


@pytest.mark.parametrize("engine_cls", ENGINES)
def test_virtual_and_empty_ops_complete_without_a_worker(engine_cls):
    w = Recorder("dp0")
    eng = engine_cls(None, Model(), None, workers={(WorkerKey(0, 0), TransferType.D2H): w})
    eng.start()
    try:
        g = TransferOpGraph()
        real = TransferOp(g.graph_id, TransferType.D2H, IDS, IDS)
        empty = TransferOp(g.graph_id, TransferType.H2DISK, IDS[:0], IDS[:0])       # no SSD worker exists
        g.add_transfer_op(real); g.add_transfer_op(empty)
        g.add_dependency(empty.op_id, real.op_id)
        v = g.add_virtual_op([real.op_id, empty.op_id])
        eng.submit(g)
        recs = drain(eng, g.graph_id)
        assert {(r.op_id, r.success) for r in recs} == {(real.op_id, True), (empty.op_id, True), (v, True), (-1, True)}
        assert w.seen == [real.op_id]
    finally:
        eng.shutdown()
