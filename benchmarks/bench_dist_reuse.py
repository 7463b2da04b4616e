#!/usr/bin/env python
"""Cross-node host reuse: node B restores prefixes that only node A's host pool holds.

Two managers with their own host pools share one registry (in-process here; a RegistryServer or a Redis
address works the same way). Node A offloads N requests; node B, which has never seen them, looks them up,
reads the blocks out of A's pool (PEERH2H), adopts them in its own host tier and restores them. Reported:
the rate of the peer read, the time of an index refresh with that many published blocks, and the second
lookup, which is served locally. Counterpart of the reference's benchmarks/benchmark_dist_kvcache.py.
Runs on a GPU (`--device cuda`) or with host stand-ins for the GPU caches (`--device cpu`).
"""
import argparse
import json
import os
import statistics
import sys
import time
import uuid

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
# only node B resets in the third round: do not wait long for node A's acknowledgement of that reset
os.environ.setdefault("FLEXKV_RESET_BARRIER_TIMEOUT_MS", "500")
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.common.transfer import TransferType  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape, make_model_config  # noqa: E402


def slots(blocks, T):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    shape = get_shape(a.model)
    T = shape.tokens_per_block
    per_req = a.tokens // T
    total_blocks = per_req * a.requests
    name = uuid.uuid4().hex
    dev = torch.device(a.device, 0) if a.device == "cuda" else "cpu"
    nodes = []
    for seed in (1, 2):
        cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=total_blocks + 64, enable_p2p_cpu=True,
                          redis_host=f"inproc:{name}")
        mgr = KVManager(make_model_config(shape), cfg, require_gpu=True)
        kv, layout = alloc_paged_cache(shape, total_blocks, dev, "vllm", fill="normal", seed=seed)
        mgr.register_gpu_tensors(kv, layout)
        mgr.start()
        mgr.wait_ready(600)
        nodes.append((mgr, kv))
    (na, kva), (nb, kvb) = nodes
    try:
        rng = np.random.default_rng(0)
        toks = [rng.integers(0, 128000, size=a.tokens, dtype=np.int64) for _ in range(a.requests)]
        pages = rng.permutation(total_blocks).reshape(a.requests, per_req)
        t0 = time.perf_counter()
        ids = [na.put_async(t, slots(p, T)) for t, p in zip(toks, pages)]
        for r in na.wait(ids, timeout=600, completely=True).values():
            assert r.status.value == "success", r.status
        put_s = time.perf_counter() - t0
        ea = na.kv_task_engine.cache_engine.cpu_cache_engine
        eb = nb.kv_task_engine.cache_engine.cpu_cache_engine
        refresh = []
        for _ in range(5):
            t0 = time.perf_counter()
            ea.refresh()
            eb.refresh()
            refresh.append((time.perf_counter() - t0) * 1e3)
        # node B: look up, bind, restore
        t0 = time.perf_counter()
        gets = []
        for t in toks:
            tid, mask = nb.get_match(t)
            assert int(mask.sum()) == a.tokens, "node B does not see node A's blocks"
            gets.append(tid)
        match_ms = (time.perf_counter() - t0) * 1e3 / a.requests
        kinds = sorted({o.transfer_type.value for tid in gets for o in nb.kv_task_engine.tasks[tid].graph.ops()})
        t0 = time.perf_counter()
        nb.launch(gets, [slots(p, T) for p in pages])
        for r in nb.wait(gets, timeout=600).values():
            assert r.status.value == "success", r.status
        get_s = time.perf_counter() - t0
        if a.device == "cuda":
            torch.cuda.synchronize()
        p0 = torch.from_numpy(pages[0])
        same = all(torch.equal(kvb[l][:, p0].cpu(), kva[l][:, p0].cpu()) for l in (0, shape.num_layers - 1))
        # second round: the blocks are B's own now
        t0 = time.perf_counter()
        again = [nb.get_match(t)[0] for t in toks]
        kinds2 = sorted({o.transfer_type.value for tid in again for o in nb.kv_task_engine.tasks[tid].graph.ops()})
        nb.launch(again, [slots(p, T) for p in pages])
        nb.wait(again, timeout=600)
        local_s = time.perf_counter() - t0
        # third round: B forgets its copies; the peer read repeats with A's pool already mapped and touched
        nb.reset_cache() if hasattr(nb, "reset_cache") else nb.reset()
        ea.refresh()
        eb.refresh()
        t0 = time.perf_counter()
        third = [nb.get_match(t)[0] for t in toks]
        kinds3 = sorted({o.transfer_type.value for tid in third for o in nb.kv_task_engine.tasks[tid].graph.ops()})
        nb.launch(third, [slots(p, T) for p in pages])
        for r in nb.wait(third, timeout=600).values():
            assert r.status.value == "success", r.status
        warm_s = time.perf_counter() - t0
        nbytes = total_blocks * shape.block_bytes
        w = nb.transfer_manager.engine.worker_for(next(iter(nb.transfer_manager.storage.gpu_regs)), TransferType.H2D)
        out = dict(benchmark="dist_host_reuse", device=a.device, model=shape.name, requests=a.requests,
                   tokens_per_request=a.tokens, blocks=total_blocks, gib=round(nbytes / 2**30, 2),
                   node_a_put_gbs=round(nbytes / put_s / 1e9, 2),
                   index_refresh_ms_p50=round(statistics.median(refresh), 2),
                   node_b_get_match_ms_per_request=round(match_ms, 3), node_b_first_get_ops=kinds,
                   node_b_first_get_gbs=round(nbytes / get_s / 1e9, 2), bytes_equal=bool(same),
                   node_b_second_get_ops=kinds2, node_b_second_get_gbs=round(nbytes / local_s / 1e9, 2),
                   node_b_third_get_after_reset_ops=kinds3, node_b_third_get_gbs=round(nbytes / warm_s / 1e9, 2),
                   h2d_worker=type(w).__name__)
        print(json.dumps(out))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(out, f)
    finally:
        nb.shutdown()
        na.shutdown()


if __name__ == "__main__":
    main()
