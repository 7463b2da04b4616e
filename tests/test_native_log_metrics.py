"""Native logger and index counters (reference: csrc/logging.cpp:50-104,
csrc/monitoring/metrics_manager.h:211-235)."""
import numpy as np
import pytest

from flexkv_b200 import _native

C = _native.C


def test_index_counters_follow_operations():
    C.configure_cpp_metrics(True)
    C.reset_cpp_metrics()
    idx = C.RadixIndex(4, 64, "lru", 0.0)
    h = np.arange(1, 9, dtype=np.uint64)
    idx.insert(np.arange(8, dtype=np.int64), h, 8, True, None)
    idx.match_prefix(h)                      # full hit
    idx.match_prefix(np.concatenate([h[:4], np.array([99], dtype=np.uint64)]))   # partial
    idx.match_prefix(np.array([1234], dtype=np.uint64))                          # miss
    idx.evict(3)
    snap = C.cpp_metrics_snapshot()
    assert snap["enabled"]
    assert snap["ops"]["insert"] == 1 and snap["blocks"]["insert"] == 8
    assert snap["ops"]["hit"] == 1 and snap["blocks"]["hit"] == 8
    assert snap["ops"]["match"] == 1 and snap["blocks"]["match"] == 4
    assert snap["ops"]["miss"] == 1
    assert snap["ops"]["evict"] == 1 and snap["blocks"]["evict"] == 3
    C.configure_cpp_metrics(False)
    idx.match_prefix(h[:5])
    assert C.cpp_metrics_snapshot()["ops"] == snap["ops"]


def test_logger_level_and_ring(capfd):
    old = C.get_log_level()
    C.set_log_level("warn")
    C.native_log(2, "should not appear")
    C.native_log(3, "disk tier degraded")
    C.set_log_level("bogus")                       # ignored
    assert C.get_log_level() == 3
    lines = C.native_log_recent(8)
    assert any("disk tier degraded" in ln and "WARN" in ln for ln in lines)
    assert not any("should not appear" in ln for ln in lines)
    C.set_log_level(["trace", "debug", "info", "warn", "error", "off"][old])


def test_prometheus_exports_native_families():
    from prometheus_client import CollectorRegistry, generate_latest
    from flexkv_b200.metrics.collector import MetricsCollector
    C.reset_cpp_metrics()
    m = MetricsCollector(CollectorRegistry())
    idx = C.RadixIndex(4, 64, "lru", 0.0)
    h = np.arange(1, 5, dtype=np.uint64)
    idx.insert(np.arange(4, dtype=np.int64), h, 4, True, None)
    text = generate_latest(m.registry).decode()
    assert 'flexkv_cpp_cache_ops_total{operation="insert"} 1.0' in text
    assert 'flexkv_cpp_cache_blocks_total{operation="insert"} 4.0' in text


def test_native_metrics_endpoint_serves_the_counters_over_http():
    """The counters of the native index have an endpoint of their own, answered by a C++ thread
    (reference: csrc/monitoring/metrics_manager.cpp:60-110, FLEXKV_CPP_METRICS_PORT)."""
    import urllib.error
    import urllib.request
    from flexkv_b200 import _native
    C = _native.C
    C.reset_cpp_metrics()
    port = C.start_cpp_metrics_exposer(0, "127.0.0.1")
    try:
        assert port > 0 and C.cpp_metrics_exposer_port() == port
        assert C.start_cpp_metrics_exposer(0, "127.0.0.1") == port          # one endpoint per process
        idx = C.RadixIndex(4, 64, "lru", 0.0)
        h = np.arange(1, 9, dtype=np.uint64)
        idx.insert(np.arange(8, dtype=np.int64), h, 8, True, None)
        idx.match_prefix(np.concatenate([h[:4], np.array([99], dtype=np.uint64)]))
        body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert "# TYPE flexkv_cpp_cache_ops_total counter" in body
        line = [l for l in body.splitlines() if l.startswith('flexkv_cpp_cache_ops_total{operation="match"}')]
        assert line and int(line[0].split()[-1]) >= 1
        assert body == C.cpp_metrics_text() or "flexkv_cpp_cache_blocks_total" in body
        with pytest.raises(urllib.error.HTTPError):
            urllib.request.urlopen(f"http://127.0.0.1:{port}/other", timeout=5)
    finally:
        C.stop_cpp_metrics_exposer()
    assert C.cpp_metrics_exposer_port() == 0
