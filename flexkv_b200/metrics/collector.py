"""Prometheus metrics (same metric names as the reference so existing dashboards
keep working: flexkv/metrics/collector.py:152-247). Enabled by
``FLEXKV_ENABLE_METRICS=1``; the HTTP endpoint listens on ``FLEXKV_PY_METRICS_PORT``."""
from __future__ import annotations

import threading
from typing import Optional

from ..common.config import GLOBAL_CONFIG_FROM_ENV
from ..common.debug import flexkv_logger

try:
    from prometheus_client import CollectorRegistry, Counter, Gauge, start_http_server
    _HAVE_PROM = True
except Exception:  # noqa: BLE001
    _HAVE_PROM = False


class MetricsCollector:
    def __init__(self, registry=None) -> None:
        if not _HAVE_PROM:
            raise RuntimeError("prometheus_client is not installed")
        self.registry = registry or CollectorRegistry()
        r = self.registry
        self.cache_hit_blocks = Counter("flexkv_py_cache_hit_blocks", "Blocks found in a tier", ["device"], registry=r)
        self.cache_miss_blocks = Counter("flexkv_py_cache_miss_blocks", "Blocks not found in a tier", ["device"],
                                         registry=r)
        self.allocation_failures = Counter("flexkv_py_allocation_failures", "Plans dropped for lack of blocks",
                                           ["device"], registry=r)
        self.transfer_blocks = Counter("flexkv_py_transfer_blocks", "Blocks moved", ["type", "operation"], registry=r)
        self.transfer_ops = Counter("flexkv_py_transfer_ops", "Transfer ops", ["type", "operation"], registry=r)
        self.transfer_bytes = Counter("flexkv_py_transfer_bytes", "Bytes moved", ["type", "operation"], registry=r)
        self.evicted_blocks = Counter("flexkv_py_evicted_blocks", "Blocks evicted", ["device"], registry=r)
        self.allocated_blocks = Counter("flexkv_py_allocated_blocks", "Blocks allocated", ["device"], registry=r)
        self.mempool_total = Gauge("flexkv_py_mempool_total_blocks", "Pool capacity", ["device"], registry=r)
        self.mempool_free = Gauge("flexkv_py_mempool_free_blocks", "Free blocks", ["device"], registry=r)
        self.peer_hit_blocks = Counter("flexkv_py_peer_gpu_hit_blocks", "Blocks pulled from a peer GPU over NVLink",
                                       registry=r)
        self._server_started = False
        self._attach_native_counters()

    def _attach_native_counters(self) -> None:
        """Expose the C++ index counters under the reference's native metric names
        (csrc/monitoring/metrics_manager.cpp:104-110); values are read at scrape time."""
        try:
            from .. import _native
            C = _native.C
        except Exception:  # noqa: BLE001
            return
        from prometheus_client.core import CounterMetricFamily

        class _Native:
            def collect(self_inner):
                snap = C.cpp_metrics_snapshot()
                ops = CounterMetricFamily("flexkv_cpp_cache_ops", "Index operations counted in native code",
                                          labels=["operation"])
                blocks = CounterMetricFamily("flexkv_cpp_cache_blocks", "Blocks touched by native index operations",
                                             labels=["operation"])
                for k, v in snap["ops"].items():
                    ops.add_metric([k], v)
                for k, v in snap["blocks"].items():
                    blocks.add_metric([k], v)
                yield ops
                yield blocks

        C.configure_cpp_metrics(True)
        self.registry.register(_Native())

    def start_server(self, port: Optional[int] = None) -> None:
        if self._server_started:
            return
        port = port or GLOBAL_CONFIG_FROM_ENV.py_metrics_port
        try:
            start_http_server(port, registry=self.registry)
            self._server_started = True
            flexkv_logger.info("metrics endpoint on :%d", port)
        except OSError as e:
            flexkv_logger.warning("metrics endpoint not started: %s", e)
        # the native counters also have an endpoint of their own, served by a C++ thread
        # (FLEXKV_CPP_METRICS_PORT, 0 switches it off; reference: csrc/monitoring/metrics_manager.cpp:60-110)
        cpp_port = int(GLOBAL_CONFIG_FROM_ENV.cpp_metrics_port or 0)
        if cpp_port > 0:
            try:
                from .. import _native
                got = _native.C.start_cpp_metrics_exposer(cpp_port)
                if got < 0:
                    flexkv_logger.warning("native metrics endpoint not started: errno %d", -got)
                else:
                    import atexit
                    atexit.register(_native.C.stop_cpp_metrics_exposer)
            except Exception as e:  # noqa: BLE001
                flexkv_logger.warning("native metrics endpoint not started: %s", e)

    def record_match(self, device: str, hit_blocks: int, miss_blocks: int) -> None:
        if hit_blocks > 0:
            self.cache_hit_blocks.labels(device).inc(hit_blocks)
        if miss_blocks > 0:
            self.cache_miss_blocks.labels(device).inc(miss_blocks)

    def record_allocation_failure(self, device: str) -> None:
        self.allocation_failures.labels(device).inc()

    def record_eviction(self, device: str, n: int) -> None:
        self.evicted_blocks.labels(device).inc(n)

    def record_transfer(self, ttype: str, blocks: int, nbytes: int, success: bool) -> None:
        op = "success" if success else "failure"
        self.transfer_ops.labels(ttype, op).inc()
        self.transfer_blocks.labels(ttype, op).inc(blocks)
        self.transfer_bytes.labels(ttype, op).inc(nbytes)
        if ttype == "PEERD2D" and success:
            self.peer_hit_blocks.inc(blocks)

    def set_mempool(self, device: str, total: int, free: int) -> None:
        self.mempool_total.labels(device).set(total)
        self.mempool_free.labels(device).set(free)

    def snapshot(self) -> dict:
        out = {}
        for fam in self.registry.collect():
            for s in fam.samples:
                if s.name.endswith("_created"):
                    continue
                out[(s.name, tuple(sorted(s.labels.items())))] = s.value
        return out


_singleton: Optional[MetricsCollector] = None
_lock = threading.Lock()


def get_collector(start_server: bool = False) -> MetricsCollector:
    global _singleton
    with _lock:
        if _singleton is None:
            _singleton = MetricsCollector()
        if start_server:
            _singleton.start_server()
        return _singleton
