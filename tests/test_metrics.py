"""Prometheus metrics through a real put/get cycle on the CPU tier and over HTTP
(metric names of the reference: flexkv/metrics/collector.py:152-247)."""
import socket
import urllib.request

import numpy as np
from prometheus_client import CollectorRegistry

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.metrics.collector import MetricsCollector
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def test_counters_follow_a_put_get_cycle_and_are_served_over_http():
    m = MetricsCollector(CollectorRegistry())
    shape = KVShape("m", 2, 2, 16, tokens_per_block=T)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=6), require_gpu=True)
    mgr.kv_task_engine.set_metrics_collector(m)
    mgr.transfer_manager.set_metrics_collector(m)
    kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=1)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    try:
        tok = np.arange(4 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots(range(4)))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        tid = mgr.get_async(tok, slots(range(10, 14)))
        assert mgr.wait(tid)[tid].status.value == "success"
        tid = mgr.put_async(tok + 100, slots(range(4, 8)))            # forces eviction: pool of 6 blocks
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        s = m.snapshot()
        block_bytes = 2 * 2 * T * 2 * 16 * 2
        assert s[("flexkv_py_transfer_blocks_total", (("operation", "success"), ("type", "D2H")))] == 8
        assert s[("flexkv_py_transfer_bytes_total", (("operation", "success"), ("type", "H2D")))] == 4 * block_bytes
        assert s[("flexkv_py_cache_hit_blocks_total", (("device", "CPU"),))] >= 4
        assert s[("flexkv_py_evicted_blocks_total", (("device", "CPU"),))] >= 2
        assert s[("flexkv_py_mempool_total_blocks", (("device", "CPU"),))] == 6
        sock = socket.socket(); sock.bind(("127.0.0.1", 0)); port = sock.getsockname()[1]; sock.close()
        m.start_server(port)
        text = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        assert "flexkv_py_transfer_ops_total" in text and "flexkv_cpp_cache_ops_total" in text
    finally:
        mgr.shutdown()
