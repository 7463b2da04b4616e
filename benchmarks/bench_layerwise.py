#!/usr/bin/env python
"""Layerwise restore benchmarks (one process drives every GPU of the group).

``--scenario notify``  the shapes of the reference's notify-mode micro-benchmark
    (MLA, kv_dim 1, 1 head, head_dim 512, fp16, 16-token blocks, contiguous ids,
    every GPU reads the same host bytes; small = 8 layers x 16 blocks, medium =
    32 x 64, large = 80 x 256): p50 time from the restore call to the last
    layer's signal, for each notify mode (benchmarks/microbenchmark_notify_mode.py:28-36,96-145).
``--scenario overlap`` Llama-3-70B TP=N in the SGLang layout (80 layers, one KV
    head per rank, 2L tensors per rank): restore of 16 x 16,384-token prefixes
    overlapped with a stand-in layer kernel of 200 us per layer that waits, in
    stream order, for its layer's KV.
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
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402

C = _native.C


HOST_LAYOUT = "blockfirst"


def build(shape, ngpu, gpu_blocks, host_blocks, engine_layout, notify, ctas, tile, tp_split, lpb=1, codec=False,
          codec_pipelines=64):
    """``codec``: the host pool holds the lossless bf16 codec's packed form (N(0,1) values packed by the offload
    kernel before the timed restores); sizes and rates are still counted in raw KV bytes."""
    regs, caches = [], []
    for d in range(ngpu):
        kv, layout = alloc_paged_cache(shape, gpu_blocks, torch.device("cuda", d), engine_layout,
                                       tp_size=ngpu if tp_split else 1, fill="normal" if codec else "zeros", seed=7 + d)
        regs.append(register_tensors(kv, layout))
        caches.append(kv)
    raw_chunk = regs[0].chunk_bytes
    chunk = raw_chunk
    if codec:
        from flexkv_b200.ops.kv_compress import chunk_slot_bytes
        chunk = chunk_slot_bytes(raw_chunk // 2)          # host slot of one chunk
    slices = ngpu if tp_split else 1
    block_bytes = slices * shape.num_layers * shape.kv_dim * chunk
    region = C.host_region_alloc(host_blocks * block_bytes, cuda_register=True, touch_threads=16,
                                 numa_node=C.gpu_numa_node(0))
    host = dict(base=region.ptr, layer_stride=shape.kv_dim * chunk, kv_stride=chunk, block_stride=block_bytes,
                num_blocks=host_blocks)
    if HOST_LAYOUT == "layerfirst" and not tp_split:
        # [layer][kv][block][chunk]: one layer of consecutive blocks is one contiguous run of host memory
        host = dict(base=region.ptr, layer_stride=shape.kv_dim * host_blocks * chunk, kv_stride=host_blocks * chunk,
                    block_stride=chunk, num_blocks=host_blocks)
    opts = dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim, chunk_bytes=raw_chunk,
                cpu_tp_stride=block_bytes // slices if tp_split else 0, shared_kv=not tp_split,
                max_blocks_per_op=max(gpu_blocks, 4096), notify_mode=notify, num_counters=3, layers_per_batch=lpb,
                h2d=dict(num_ctas=ctas, tile_bytes=tile, engine=0))
    if codec:
        from flexkv_b200.ops.kv_compress import kv_compress, tiles_per_chunk
        from flexkv_b200.ops.kv_copy import HostSide, decode_status, new_status
        L, K, tpc = shape.num_layers, shape.kv_dim, tiles_per_chunk(raw_chunk // 2)
        per_rank = L * K * tpc
        table = torch.zeros(host_blocks * slices * per_rank, dtype=torch.int32).pin_memory()
        ids = np.arange(min(gpu_blocks, host_blocks), dtype=np.int64)
        for d, reg in enumerate(regs if tp_split else regs[:1]):
            with torch.cuda.device(d):
                st = new_status(torch.device("cuda", d))
                hs = HostSide(region.ptr, host["layer_stride"], host["kv_stride"], block_bytes, host_blocks,
                              offset=d * (block_bytes // slices) if tp_split else 0)
                off = d * per_rank if tp_split else 0
                keep = kv_compress(reg, hs, table[off:], ids, ids, h2d=False, layers_total=slices * L, num_ctas=64,
                                   status=st)
                torch.cuda.synchronize(d)
                assert decode_status(st) == 0
                del keep
        used = table[table > 0].double()
        opts.update(size_table_ptr=table.data_ptr(), size_table_layers=slices * L,
                    size_table_rank_entries=per_rank if tp_split else 0, codec_pipelines=codec_pipelines)
        build.packed_ratio = float(used.sum()) / (used.numel() * 2.0 * min(8192, raw_chunk // 2)) if used.numel() else 0
        build.table = table
    grp = C.LayerwiseGroup([r.as_native() for r in regs], host, opts)
    return grp, region, caches, raw_chunk, block_bytes


def scenario_notify(a):
    out = []
    scales = {"small": (8, 16), "medium": (32, 64), "large": (80, 256)}
    modes = [("hostfunc", 1), ("polling", 1), ("flag", 1), ("flag", 0)]
    if a.modes:
        modes = [m for m in modes if (m[0] + ("+fused" if m[1] == 0 else "")) in a.modes]
    for name, (layers, blocks) in scales.items():
        if a.scales and name not in a.scales:
            continue
        shape = KVShape(name, layers, 1, 512, dtype=torch.float16, use_mla=True, tokens_per_block=16)
        for notify, lpb in modes:
            grp, region, caches, chunk, bb = build(shape, a.gpus, blocks, blocks, "vllm", notify, a.ctas or 4,
                                                   a.tile_bytes, tp_split=False, lpb=lpb)
            ids = np.arange(blocks, dtype=np.int64)
            lat = []
            for i in range(a.iters + 5):
                for d in range(a.gpus):
                    torch.cuda.synchronize(d)
                t0 = time.perf_counter()
                r = grp.restore(ids, ids, i % 3)
                dt = (time.perf_counter() - t0) * 1e3
                assert r.status == 0
                if i >= 5:
                    lat.append(dt)
            p50 = statistics.median(lat)
            per_gpu = layers * blocks * chunk
            row = dict(scale=name, notify=notify + ("+fused" if lpb == 0 else ""), gpus=a.gpus, p50_ms=round(p50, 3),
                       gbs_per_gpu=round(per_gpu / p50 / 1e6, 2), bytes_per_gpu=per_gpu,
                       gpu_ms=round(r.total_ms, 3), host_layout=HOST_LAYOUT)
            out.append(row)
            print(json.dumps(row), flush=True)
            del grp
            region.free()
    return out


def scenario_overlap(a):
    shape = KVShape("llama3-70b", 80, 8, 128, tokens_per_block=16)
    nblocks = a.requests * a.tokens // 16
    grp, region, caches, chunk, bb = build(shape, a.gpus, nblocks, nblocks, "sglang", a.notify, a.ctas or 8,
                                           a.tile_bytes, tp_split=a.gpus > 1, lpb=a.layers_per_batch, codec=a.codec,
                                           codec_pipelines=a.codec_pipelines)
    L = shape.num_layers
    rng = np.random.default_rng(0)
    cpu = rng.permutation(nblocks).astype(np.int64)
    streams = [torch.cuda.Stream(device=d) for d in range(a.gpus)]
    busy_ns = int(a.layer_us * 1000)
    rows = []
    import threading
    for it in range(a.iters + 2):
        gpu = rng.permutation(nblocks).astype(np.int64)
        counter = it % 3
        for d in range(a.gpus):
            torch.cuda.synchronize(d)
        evs = []
        t0 = time.perf_counter()
        res = {}
        epoch = grp.begin_restore(counter)     # the value this round's restore will publish to the layer flags
        th = threading.Thread(target=lambda: res.setdefault("r", grp.restore(gpu, cpu, counter)))
        th.start()
        # the waits go to the GPU only after the restore's launches are queued: a stream wait ahead of its producer
        # can block the hardware queue they share
        assert grp.wait_launched(counter, epoch, 30000), "the restore did not queue its launches"
        # the model: per layer, wait (in stream order) for the layer's KV, then "compute"
        for d in range(a.gpus):
            with torch.cuda.device(d):
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record(streams[d])
                for l in range(L):
                    grp.stream_wait_layer(d, counter, l, streams[d].cuda_stream, epoch)
                    C.layer_stub(0, 0, busy_ns, 0, 0, 0, a.stub_ctas, streams[d].cuda_stream)
                e1.record(streams[d])
                evs.append((e0, e1))
        th.join()
        for d in range(a.gpus):
            torch.cuda.synchronize(d)
        wall = (time.perf_counter() - t0) * 1e3
        r = res["r"]
        assert r.status == 0
        model_ms = max(e0.elapsed_time(e1) for e0, e1 in evs)
        if it >= 2:
            rows.append((r.total_ms, model_ms, wall))
    restore_ms = statistics.median(x[0] for x in rows)
    model_ms = statistics.median(x[1] for x in rows)
    per_rank = nblocks * L * shape.kv_dim * chunk
    row = dict(scenario="overlap", gpus=a.gpus, notify=a.notify,
               host_pool="bf16_xp packed, %.3f of raw" % build.packed_ratio if a.codec else "raw", layers_per_batch=a.layers_per_batch, blocks=nblocks, bytes_per_rank=per_rank,
               restore_ms=round(restore_ms, 2), restore_gbs_per_gpu=round(per_rank / restore_ms / 1e6, 2),
               restore_gbs_box=round(a.gpus * per_rank / restore_ms / 1e6, 2),
               compute_only_ms=round(L * a.layer_us / 1e3, 2), overlapped_total_ms=round(model_ms, 2),
               serial_sum_ms=round(restore_ms + L * a.layer_us / 1e3, 2),
               wall_ms=round(statistics.median(x[2] for x in rows), 2))
    print(json.dumps(row), flush=True)
    return [row]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenario", default="notify", choices=["notify", "overlap"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--tile-bytes", type=int, default=16384)
    ap.add_argument("--notify", default="flag")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--layer-us", type=float, default=200.0)
    ap.add_argument("--stub-ctas", type=int, default=148)
    ap.add_argument("--layers-per-batch", type=int, default=0, help="0 = one fused launch with per-layer flags")
    ap.add_argument("--out", default="")
    ap.add_argument("--codec", action="store_true", help="overlap: host pool in the lossless codec's packed form")
    ap.add_argument("--codec-pipelines", type=int, default=64)
    ap.add_argument("--host-layout", default="blockfirst", choices=["blockfirst", "layerfirst"],
                    help="host pool layout (FLEXKV_CPU_LAYOUT of a deployment)")
    ap.add_argument("--scales", nargs="*", default=[], help="notify: subset of small medium large")
    ap.add_argument("--modes", nargs="*", default=[], help="notify: subset of hostfunc polling flag flag+fused")
    a = ap.parse_args()
    global HOST_LAYOUT
    HOST_LAYOUT = a.host_layout
    rows = scenario_notify(a) if a.scenario == "notify" else scenario_overlap(a)
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
