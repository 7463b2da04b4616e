#!/usr/bin/env python
"""Both PCIe directions at once: a GPU->host and a host->GPU paged copy (disjoint random blocks,
2048 Llama-3-8B blocks = 4 GiB each) issued together on two transfer groups, over CTA counts and
tile sizes, against the same pair of contiguous copies on the copy engines.

    python benchmarks/bench_duplex.py [out.json]

Per row: wall time of the overlapped pair (host clock between two device synchronisations) and the
sum of both directions' bytes over it; the kernels' own CUDA-event times are listed beside it.
"""
import json
import os
import sys
import threading
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402

C = _native.C


def main() -> None:
    dev = torch.device("cuda:0")
    shape = get_shape("llama3-8b")
    NB, n = 4096, 2048
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=1)
    reg = register_tensors(kv, layout)
    bb = shape.block_bytes
    region = C.host_region_alloc(NB * bb, numa_node=C.gpu_numa_node(0), cuda_register=True, touch_threads=16)
    chunk = reg.chunk_bytes
    host = dict(base=region.ptr, layer_stride=2 * chunk, kv_stride=chunk, block_stride=bb, num_blocks=NB)
    opts = dict(num_layers=shape.num_layers, kv_dim=2, chunk_bytes=chunk, max_blocks_per_op=NB)
    g_out, g_in = C.TransferGroup([reg.as_native()], host, opts), C.TransferGroup([reg.as_native()], host, opts)
    rng = np.random.default_rng(0)
    rows = []

    def pair(fn_a, fn_b, reps=3):
        best, parts = 1e9, None
        for r in range(reps + 1):
            res = {}
            ths = [threading.Thread(target=lambda: res.__setitem__("a", fn_a())),
                   threading.Thread(target=lambda: res.__setitem__("b", fn_b()))]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for t in ths:
                t.start()
            for t in ths:
                t.join()
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) * 1e3
            if r > 0 and dt < best:
                best, parts = dt, (res["a"], res["b"])
        return best, parts

    # the router's staged route: scattered GPU pages, host blocks in two runs (what a fresh allocation gives): the
    # kernel gathers into device staging, the copy engines cross the link, one direction per engine
    g_out.set_launch(False, 8, 16384, 3)
    g_in.set_launch(True, 8, 16384, 3)
    gp = rng.permutation(NB)
    ga, gb = gp[:n].astype(np.int64), gp[n:2 * n].astype(np.int64)
    ca, cb = np.arange(0, n, dtype=np.int64), np.arange(n, 2 * n, dtype=np.int64)

    def d2h_staged():
        o = g_out.transfer(ga, ca, False, 0, shape.num_layers)
        assert o.status == 0, o.status
        return o.gpu_ms

    def h2d_staged():
        o = g_in.transfer(gb, cb, True, 0, shape.num_layers)
        assert o.status == 0, o.status
        return o.gpu_ms
    ms, (m_out, m_in) = pair(d2h_staged, h2d_staged)
    row = dict(engine="router: gather into staging + copy engines (host blocks in runs)", pair_ms=round(ms, 2),
               both_gbs=round(2 * n * bb / ms / 1e6, 2), d2h_gbs=round(n * bb / m_out / 1e6, 2),
               h2d_gbs=round(n * bb / m_in / 1e6, 2), staged_ops=[int(g_out.staged_ops), int(g_in.staged_ops)])
    rows.append(row)
    print(json.dumps(row), flush=True)

    for engine, name in ((0, "tma"), (1, "simt")):
        if "--staged-only" in sys.argv:
            break
        for ctas in (4, 8, 16, 32, 64):
            for tile in ((8192, 16384, 32768) if engine == 0 else (16384,)):
                g_out.set_launch(False, ctas, tile, engine)
                g_in.set_launch(True, ctas, tile, engine)
                gp, cp = rng.permutation(NB), rng.permutation(NB)
                ga, gb = gp[:n].astype(np.int64), gp[n:2 * n].astype(np.int64)
                ca, cb = cp[:n].astype(np.int64), cp[n:2 * n].astype(np.int64)

                def d2h():
                    o = g_out.transfer(ga, ca, False, 0, shape.num_layers)
                    assert o.status == 0, o.status
                    return o.gpu_ms

                def h2d():
                    o = g_in.transfer(gb, cb, True, 0, shape.num_layers)
                    assert o.status == 0, o.status
                    return o.gpu_ms
                ms, (m_out, m_in) = pair(d2h, h2d)
                row = dict(engine=name, ctas=ctas, tile=tile, pair_ms=round(ms, 2),
                           both_gbs=round(2 * n * bb / ms / 1e6, 2), d2h_gbs=round(n * bb / m_out / 1e6, 2),
                           h2d_gbs=round(n * bb / m_in / 1e6, 2))
                rows.append(row)
                print(json.dumps(row), flush=True)

    # the copy engines on the same byte counts, contiguous
    nbytes = n * bb
    pin_a, pin_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_a, d_b = torch.empty(nbytes, dtype=torch.uint8, device=dev), torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    best = 1e9
    for r in range(4):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.cuda.stream(s1):
            pin_a.copy_(d_a, non_blocking=True)
        with torch.cuda.stream(s2):
            d_b.copy_(pin_b, non_blocking=True)
        torch.cuda.synchronize()
        if r > 0:
            best = min(best, (time.perf_counter() - t0) * 1e3)
    row = dict(engine="copy engines, contiguous", pair_ms=round(best, 2), both_gbs=round(2 * nbytes / best / 1e6, 2))
    rows.append(row)
    print(json.dumps(row), flush=True)
    if len(sys.argv) > 1 and not sys.argv[1].startswith("--"):
        os.makedirs(os.path.dirname(os.path.abspath(sys.argv[1])), exist_ok=True)
        with open(sys.argv[1], "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
