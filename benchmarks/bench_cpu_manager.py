#!/usr/bin/env python
"""CPU-only KVManager workload: put-then-get over a host pool plus a file-backed SSD
tier with radix-tree prefix matching; no GPU involved (the engine's paged cache is a
host tensor and the data plane copies with CPU threads).

Llama-3-8B KV shape (32 layers, 8 KV heads, head 128, bf16, 16-token blocks = 2 MiB per
block). 1,000 requests of 1,024-8,192 tokens (uniform, seeded), token ids uniform in
[0, 128256); half of the requests start with one of 64 shared random prefixes of
512-4,096 tokens; KV values N(0,1). Host pool 4 GiB, SSD pool 16 GiB, world size 1.
Every request is first looked up (get of whatever prefix is cached), then put.
Reports control-plane latencies (hash + match + plan), hit rates and data-plane GB/s.
"""
import argparse
import json
import os
import statistics
import sys
import tempfile
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape, make_model_config  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=1000)
    ap.add_argument("--cpu-gib", type=float, default=4.0)
    ap.add_argument("--ssd-gib", type=float, default=16.0)
    ap.add_argument("--ssd-dir", default="")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--index", default="native", choices=["native", "python"])
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    if a.index == "python":
        from flexkv_b200.common.config import GLOBAL_CONFIG_FROM_ENV
        GLOBAL_CONFIG_FROM_ENV.index_accel = False

    shape = get_shape("llama3-8b")
    T, bb = shape.tokens_per_block, shape.block_bytes
    ssd_dir = a.ssd_dir or tempfile.mkdtemp(prefix="flexkv_ssd_")
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=int(a.cpu_gib * 2**30) // bb, enable_ssd=a.ssd_gib > 0,
                      num_ssd_blocks=max(1, int(a.ssd_gib * 2**30) // bb), ssd_cache_dir=ssd_dir)
    mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
    NB = 1024                                                   # stand-in paged cache: 2 GiB, fits two 8K requests
    kv, layout = alloc_paged_cache(shape, NB, "cpu", "vllm", fill="normal", seed=a.seed)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(600)

    rng = np.random.default_rng(a.seed)
    prefixes = [rng.integers(0, 128256, size=int(rng.integers(512, 4097)), dtype=np.int64) for _ in range(64)]
    t_match, t_put_plan, get_ms, put_ms = [], [], [], []
    get_bytes = put_bytes = 0
    hit_tokens = query_tokens = 0
    t_all = time.perf_counter()
    for i in range(a.requests):
        n = int(rng.integers(1024, 8193))
        body = rng.integers(0, 128256, size=n, dtype=np.int64)
        if rng.random() < 0.5:
            pre = prefixes[int(rng.integers(64))]
            tok = np.concatenate([pre, body])[:n] if len(pre) < n else pre[:n].copy()
        else:
            tok = body
        nblk = n // T
        blocks = rng.permutation(NB)[:nblk].astype(np.int64)
        slot = np.repeat(blocks, T) * T + np.tile(np.arange(T), nblk)
        # lookup + restore of whatever is cached
        t0 = time.perf_counter()
        tid, mask = mgr.get_match(tok[:nblk * T])
        t_match.append((time.perf_counter() - t0) * 1e3)
        hit = int(mask.sum())
        hit_tokens += hit
        query_tokens += nblk * T
        if hit:
            t0 = time.perf_counter()
            mgr.launch(tid, slot[:hit])
            r = mgr.wait(tid, timeout=120)[tid]
            get_ms.append((time.perf_counter() - t0) * 1e3)
            assert r.status.value == "success", r
            get_bytes += hit * shape.bytes_per_token
        # offload
        t0 = time.perf_counter()
        tid, mask = mgr.put_match(tok[:nblk * T])
        t_put_plan.append((time.perf_counter() - t0) * 1e3)
        new = int(mask.sum())
        if new:
            t0 = time.perf_counter()
            mgr.launch(tid, slot[mask])
            r = mgr.wait(tid, timeout=120, completely=True)[tid]
            put_ms.append((time.perf_counter() - t0) * 1e3)
            assert r.status.value == "success", r
            put_bytes += new * shape.bytes_per_token
    wall = time.perf_counter() - t_all
    eng = mgr.kv_task_engine.cache_engine
    out = {
        "benchmark": "cpu_only_kvmanager", "requests": a.requests, "index": a.index, "wall_s": round(wall, 2),
        "get_match_ms_p50": round(statistics.median(t_match), 3),
        "get_match_ms_p99": round(sorted(t_match)[int(0.99 * (len(t_match) - 1))], 3),
        "put_match_ms_p50": round(statistics.median(t_put_plan), 3),
        "token_hit_rate": round(hit_tokens / max(1, query_tokens), 4),
        "get_gbs": round(get_bytes / max(1e-9, sum(get_ms) / 1e3) / 1e9, 2),
        "put_gbs_incl_ssd_write": round(put_bytes / max(1e-9, sum(put_ms) / 1e3) / 1e9, 2),
        "get_gib": round(get_bytes / 2**30, 2), "put_gib": round(put_bytes / 2**30, 2),
        "cpu_evicted_blocks": eng.cpu_cache_engine.num_evicted_total,
        "ssd_evicted_blocks": eng.ssd_cache_engine.num_evicted_total if eng.ssd_cache_engine else 0,
        "ssd_io": "io_uring" if mgr.transfer_manager.storage.ssd and
        mgr.transfer_manager.storage.ssd.engine.using_iouring else "threads",
    }
    print(json.dumps(out))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    mgr.shutdown()


if __name__ == "__main__":
    main()
