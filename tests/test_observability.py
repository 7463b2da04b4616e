"""Structured logs: ``[XFER]`` per-op records and ``[XFER-SUMMARY]`` percentiles from a live manager,
the ``operation=... act=... status=...`` line format and the batching of eviction events
(reference: tests/test_transfer_trace.py, tests/test_operational_logging.py,
flexkv/transfer/trace.py:134-199, flexkv/common/debug.py)."""
import re

import numpy as np

from flexkv_b200.common.debug import EvictionLogAggregator, format_op_log
from flexkv_b200.models import KVShape
from flexkv_b200.transfer.trace import TransferTrace

from test_kvmanager_cpu import slots, start

XFER = re.compile(r"^\[XFER\] op=(\d+) type=(\w+) blocks=(\d+) bytes=(\d+) wait_ms=([\d.]+) xfer_ms=([\d.]+) "
                  r"e2e_ms=([\d.]+) bw_GBps=([\d.]+) ok=([01])$")
SUMMARY = re.compile(r"^\[XFER-SUMMARY\] type=(\w+) n=(\d+) p50_ms=([\d.]+) p99_ms=([\d.]+) bw_p50_GBps=([\d.]+)$")


def test_transfer_trace_records_every_op_of_a_put_and_a_get(tmp_path):
    shape = KVShape("t", 2, 2, 16, tokens_per_block=4)
    mgr, (kv,) = start(shape, "vllm", num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=64,
                       ssd_cache_dir=str(tmp_path))
    try:
        trace = mgr.transfer_manager.engine._trace
        trace.enabled = True
        tok = np.arange(6 * 4, dtype=np.int64)
        tid = mgr.put_async(tok, slots(range(6), 4))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        mgr._clear_cpu_cache()
        tid = mgr.get_async(tok, slots(range(10, 16), 4))
        assert mgr.wait(tid)[tid].status.value == "success"
        recs = [XFER.match(l) for l in trace.lines]
        assert all(recs) and len(recs) == 4
        by_type = {m.group(2): m for m in recs}
        assert set(by_type) == {"D2H", "H2DISK", "DISK2H", "H2D"}
        block_bytes = mgr.transfer_manager.storage.host.block_bytes
        for m in recs:
            assert int(m.group(3)) == 6 and int(m.group(4)) == 6 * block_bytes and m.group(9) == "1"
            assert float(m.group(7)) + 1e-3 >= float(m.group(6))           # e2e covers the transfer itself
        out = trace.summary()
        got = {SUMMARY.match(l).group(1): int(SUMMARY.match(l).group(2)) for l in out}
        assert got == {"D2H": 1, "H2DISK": 1, "DISK2H": 1, "H2D": 1}
        assert trace.summary() == []                                         # a summary starts a new window
    finally:
        mgr.shutdown()


def test_disabled_trace_keeps_nothing():
    class Op:
        op_id = 1
    t = TransferTrace(enabled=False)
    t.on_submit(Op())
    t.on_done(Op(), None)
    assert t.lines == [] and t.summary() == []


def test_operation_line_format_and_eviction_batching():
    assert format_op_log("put", "launch", "ok", task_id=3, blocks=7) == \
        "operation=put act=launch status=ok task_id=3 blocks=7"
    agg = EvictionLogAggregator(interval_s=3600.0)
    assert agg.record("CPU", 5) is None and agg.record("CPU", 2) is None and agg.record("SSD", 1) is None
    assert agg.flush() == "operation=evict act=aggregate status=ok detail=CPU:blocks=7,events=2 SSD:blocks=1,events=1"
    assert agg.flush() is None
    agg = EvictionLogAggregator(interval_s=0.0)
    assert agg.record("CPU", 4) == "operation=evict act=aggregate status=ok detail=CPU:blocks=4,events=1"


def test_an_eviction_that_cannot_make_room_warns_at_once(caplog):
    import logging
    import numpy as np
    from flexkv_b200.cache.cache_engine import CacheEngine
    from flexkv_b200.common.block import SequenceMeta
    from flexkv_b200.common.transfer import DeviceType
    e = CacheEngine(DeviceType.CPU, 4, 4)
    s = SequenceMeta(np.arange(16, dtype=np.int64), 4)
    node = e.insert(s, e.take(4), is_ready=True)
    e.lock_node(node)                                   # everything cached is pinned by a running transfer
    with caplog.at_level(logging.WARNING, logger="flexkv"):
        got = e.take(2, strict=False)
    assert len(got) == 0
    lines = [r.getMessage() for r in caplog.records if "operation=eviction" in r.getMessage()]
    assert lines and "act=batch status=target_miss" in lines[0] and "tier=CPU" in lines[0] and "wanted=2" in lines[0]
    assert "target_met=false" in lines[0]
    e.unlock(node)
    caplog.clear()
    with caplog.at_level(logging.WARNING, logger="flexkv"):
        assert len(e.take(2, strict=False)) == 2       # now the eviction makes room: no warning
    assert not [r for r in caplog.records if "target_miss" in r.getMessage()]
