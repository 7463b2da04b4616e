#!/usr/bin/env python
"""Throughput of each transfer worker on its own: GPU<->host, host<->SSD and (with --gds)
SSD<->GPU, driven with synthetic ops through the worker's own ``execute`` — no planner, no
index (the reference's script of this name times its worker processes the same way,
benchmarks/benchmark_workers.py).

    python benchmarks/benchmark_workers.py [--config benchmarks/example_config.yml] \
        [--blocks 1024] [--iters 5] [--ssd-dir /tmp/flexkv_bench] [--gds] [--out rows.json]

Every row: worker, blocks per op, bytes per op, p50 over ``--iters`` ops of the host clock around
``execute`` (which returns when the bytes have landed), and the GPU-event time where the worker
reports one. Block ids are random permutations, the same for every worker.
"""
import argparse
import json
import os
import statistics
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.common.transfer import TransferOp, TransferType, WorkerKey  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache  # noqa: E402

from benchmark_single_batch import load  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(os.path.dirname(__file__), "example_config.yml"))
    ap.add_argument("--blocks", type=int, default=1024, help="blocks per op")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--ssd-dir", default="")
    ap.add_argument("--gds", action="store_true")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    model, cache, _ = load(a.config)
    n = a.blocks
    cache.num_cpu_blocks = 2 * n
    cache.enable_ssd = bool(a.ssd_dir)
    if a.ssd_dir:
        cache.ssd_cache_dir = a.ssd_dir
        cache.num_ssd_blocks = 2 * n
        cache.enable_gds = bool(a.gds)
    T = cache.tokens_per_block
    shape = KVShape("bench", model.num_layers, model.num_kv_heads, model.head_size, dtype=model.dtype,
                    use_mla=model.use_mla, tokens_per_block=T)
    dev = a.device if a.device == "cpu" else torch.device(a.device)
    mgr = KVManager(model, cache, require_gpu=True, in_process=True)
    kv, layout = alloc_paged_cache(shape, 2 * n, dev, "vllm", tp_size=model.tp_size, fill="normal")
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(600)
    rows = []
    try:
        workers = mgr.transfer_manager.engine._workers
        block_bytes = mgr.transfer_manager.storage.host.block_bytes
        rng = np.random.default_rng(0)
        gpu, cpu, ssd = (rng.permutation(2 * n)[:n].astype(np.int64) for _ in range(3))
        plan = [(TransferType.D2H, gpu, cpu), (TransferType.H2D, cpu, gpu),
                (TransferType.H2DISK, cpu, ssd), (TransferType.DISK2H, ssd, cpu),
                (TransferType.D2DISK, gpu, ssd), (TransferType.DISK2D, ssd, gpu)]
        for tt, src, dst in plan:
            w = workers.get((WorkerKey(0, 0), tt))
            if w is None:
                continue
            wall, dev_ms = [], []
            for i in range(a.warmup + a.iters):
                op = TransferOp(0, tt, src, dst)
                if a.device != "cpu":
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                out = w.execute(op)
                dt = (time.perf_counter() - t0) * 1e3
                if not out.success:
                    raise RuntimeError(f"{tt.value}: {out.error}")
                if i >= a.warmup:
                    wall.append(dt)
                    dev_ms.append(out.gpu_ms)
            p50 = statistics.median(wall)
            g50 = statistics.median(dev_ms)
            row = dict(worker=getattr(w, "name", type(w).__name__), type=tt.value, blocks=n,
                       bytes=n * block_bytes, p50_ms=round(p50, 3), gbs=round(n * block_bytes / p50 / 1e6, 2),
                       gpu_event_ms=round(g50, 3),
                       gbs_gpu_events=round(n * block_bytes / g50 / 1e6, 2) if g50 > 0 else None)
            rows.append(row)
            print(json.dumps(row), flush=True)
    finally:
        mgr.shutdown()
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
