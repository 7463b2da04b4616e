#!/usr/bin/env python
"""Control-plane micro-benchmarks on the CPU (no GPU involved).

* hashing: cumulative XXH64 block keys of 8K-token sequences, one sequence at a time and
  batched over threads (native), against a pure-Python restatement of the same digest chain;
* index: insert / match / evict of 512-block sequences with 50 % shared prefixes on the native
  radix index and on the Python specification index (same calls, same data);
* planner + scheduler: put then get of 8K-token requests through KVTaskEngine with a data plane
  whose workers complete at once, i.e. the per-request cost of hash + match + plan + graph
  scheduling + completion.
(Reference counterparts: benchmarks/benchmark_cache_engine.py, microbenchmark_transfer_scheduler.py.)
"""
import argparse
import json
import os
import statistics
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.cache.radixtree import RadixTreeIndex  # noqa: E402

C = _native.C
T = 16


def bench_hash(a):
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 128256, size=8192, dtype=np.int64) for _ in range(64)]
    t0 = time.perf_counter()
    for _ in range(a.reps):
        for s in seqs:
            C.gen_hashes(s, T, None)
    one = (time.perf_counter() - t0) / (a.reps * len(seqs))
    t0 = time.perf_counter()
    for _ in range(a.reps):
        C.gen_hashes_batch(seqs, T, None, 8)
    batch = (time.perf_counter() - t0) / (a.reps * len(seqs))
    # the same digest chain in Python over the native one-shot hash (what a Python control plane would do
    # without streaming state: re-hash the whole prefix per block is quadratic, so hash block by block instead)
    t0 = time.perf_counter()
    for s in seqs[:4]:
        for i in range(len(s) // T):
            C.xxh64(s[i * T:(i + 1) * T], 0)
    py = (time.perf_counter() - t0) / 4
    return dict(bench="hash_8k_tokens", native_us=round(one * 1e6, 1), native_batched_us_per_seq=round(batch * 1e6, 1),
                python_loop_us=round(py * 1e6, 1), native_tokens_per_s=round(8192 / one / 1e6, 1),
                unit_tokens_per_s="M tokens/s")


def _workload(n, seed=0):
    rng = np.random.default_rng(seed)
    prefixes = [rng.integers(1, 2**62, size=256, dtype=np.uint64) for _ in range(32)]
    out = []
    for i in range(n):
        body = rng.integers(1, 2**62, size=512, dtype=np.uint64)
        if i % 2:
            body[:256] = prefixes[i % 32]
        out.append(body)
    return out


def bench_index(a):
    rows = []
    seqs = _workload(a.index_seqs)
    for name, make in (("native", lambda: C.RadixIndex(T, 0, "lru", 0.0)),
                       ("python", lambda: RadixTreeIndex(T, 0, "lru", 0.0))):
        idx = make()
        next_block = 0
        t_ins, t_match = [], []
        for h in seqs:
            t0 = time.perf_counter()
            m = idx.match_prefix(h, len(h), True) if name == "native" else idx.match_prefix(h, len(h), True)
            t_match.append(time.perf_counter() - t0)
            need = len(h) - m.num_matched_blocks
            phys = np.arange(next_block, next_block + need, dtype=np.int64)
            next_block += need
            t0 = time.perf_counter()
            idx.insert(phys, h, len(h), True, m)
            t_ins.append(time.perf_counter() - t0)
        t0 = time.perf_counter()
        for h in seqs:
            idx.match_prefix(h, len(h), True)
        t_hit = (time.perf_counter() - t0) / len(seqs)
        t0 = time.perf_counter()
        total = 0
        while True:
            ev = idx.evict(4096)
            n = len(ev[0])
            total += n
            if n == 0:
                break
        t_ev = time.perf_counter() - t0
        rows.append(dict(bench="index_512_blocks", index=name, match_miss_us=round(statistics.median(t_match) * 1e6, 1),
                         insert_us=round(statistics.median(t_ins) * 1e6, 1), match_hit_us=round(t_hit * 1e6, 1),
                         evict_blocks_per_ms=round(total / max(t_ev, 1e-9) / 1e3, 1), blocks=total))
    return rows


def bench_planner(a, instant_workers=True):
    """``instant_workers``: the workers report success without touching memory, so the figure is hash + match +
    plan + graph scheduling + two thread hops + completion and nothing else. With False the CPU stand-in of the
    copy kernel runs too (1 024 scattered 256-byte copies into a 64 MiB pool per request: cache misses, not control plane)."""
    from flexkv_b200 import CacheConfig, KVManager
    from flexkv_b200.models import alloc_paged_cache, KVShape, make_model_config
    from flexkv_b200.transfer import workers as W
    shape = KVShape("tiny", 1, 1, 8, tokens_per_block=T)     # 256 B blocks
    saved = W.HostEmulatedGpuWorker.execute
    if instant_workers:
        W.HostEmulatedGpuWorker.execute = lambda self, op: W.OpOutcome(True, num_bytes=0)
    try:
        mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=max(1 << 17, a.requests * 512)),
                        require_gpu=True)      # every put stays resident: every get is a full hit
        kv, layout = alloc_paged_cache(shape, 4096, "cpu", "vllm", fill="zeros")
        mgr.register_gpu_tensors(kv, layout)
        mgr.start(); mgr.wait_ready(60)
        rng = np.random.default_rng(1)
        put_ms, get_ms = [], []
        slot = np.arange(8192, dtype=np.int64)
        toks = [rng.integers(0, 128256, size=8192, dtype=np.int64) for _ in range(a.requests)]
        for tok in toks:
            t0 = time.perf_counter()
            tid = mgr.put_async(tok, slot)
            mgr.wait(tid, completely=True)
            put_ms.append((time.perf_counter() - t0) * 1e3)
        for tok in toks:
            t0 = time.perf_counter()
            tid, mask = mgr.get_match(tok)
            mgr.launch(tid, slot[mask])
            mgr.wait(tid)
            get_ms.append((time.perf_counter() - t0) * 1e3)
        mgr.shutdown()
    finally:
        W.HostEmulatedGpuWorker.execute = saved
    p99 = lambda v: round(sorted(v)[int(0.99 * (len(v) - 1))], 3)
    return dict(bench="plan_and_schedule_8k_request", workers="instant" if instant_workers else "host copy stand-in",
                put_ms_p50=round(statistics.median(put_ms), 3), put_ms_p99=p99(put_ms),
                get_ms_p50=round(statistics.median(get_ms), 3), get_ms_p99=p99(get_ms), requests=a.requests)


def bench_warm_restart(a):
    """Image of a large SSD index: export, import into an empty index, reservation of its blocks."""
    import io
    from flexkv_b200 import _native
    C = _native.C
    N = 1_000_000
    idx = C.RadixIndex(T, N, "lru", 0.0, 2)
    rng = np.random.default_rng(0)
    prefixes = [rng.integers(1, 2**63, size=128, dtype=np.int64).astype(np.uint64) for _ in range(64)]
    nxt = 0
    for i in range(1950):
        s = np.concatenate([prefixes[i % 64], rng.integers(1, 2**63, size=384, dtype=np.int64).astype(np.uint64)])
        m = idx.match_prefix(s, len(s), False)
        need = len(s) - m.num_matched_blocks
        idx.insert(np.arange(nxt, nxt + need, dtype=np.int64), s, len(s), True, m)
        nxt += need
    t_exp, t_imp, t_res = [], [], []
    for _ in range(a.reps):
        t0 = time.perf_counter()
        img = idx.export_ready()
        t1 = time.perf_counter()
        other = C.RadixIndex(T, N, "lru", 0.0, 2)
        n = other.import_snapshot(*img)
        t2 = time.perf_counter()
        pool = C.BlockPool(N)
        pool.reserve(img[3])
        t3 = time.perf_counter()
        t_exp.append(t1 - t0); t_imp.append(t2 - t1); t_res.append(t3 - t2)
    buf = io.BytesIO()
    np.savez(buf, parents=img[0], sizes=img[1], hashes=img[2], blocks=img[3])
    return dict(bench="ssd_index_image", blocks=int(n), nodes=int(idx.num_nodes()),
                export_ms=round(statistics.median(t_exp) * 1e3, 1), import_ms=round(statistics.median(t_imp) * 1e3, 1),
                reserve_ms=round(statistics.median(t_res) * 1e3, 1), image_mb=round(buf.tell() / 1e6, 1))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--index-seqs", type=int, default=400)
    ap.add_argument("--requests", type=int, default=200)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rows = [bench_hash(a)] + bench_index(a) + [bench_planner(a, True), bench_planner(a, False), bench_warm_restart(a)]
    for r in rows:
        print(json.dumps(r))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
