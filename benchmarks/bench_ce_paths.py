#!/usr/bin/env python
"""Copy-engine router against the TMA kernel as a function of run length.

Llama-3-8B blocks (32 layers x K/V x 32 KiB chunks, vLLM layer-first GPU layout, block-first
host pool), 8 GiB per direction and point. Block ids are laid out as runs of ``run`` consecutive
(gpu, cpu) ids at random positions: run 1 is the scattered case of the headline benchmark, run
512 is one 8K-token request in contiguous pages. For every run length the op is timed with the
kernel (engine tma), forced copy engine (ce) and the router (auto), CUDA events, 3 warm-ups.
(Reference counterpart: benchmarks/microbenchmark_ce_strategy.py, microbenchmark_ce_threshold.py.)
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402

ENG = {"tma": 0, "ce": 2, "auto": 3}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=4096, help="blocks per op (2 MiB each)")
    ap.add_argument("--runs", type=int, nargs="+", default=[1, 4, 16, 64, 512])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    shape = get_shape("llama3-8b")
    NB = 2 * a.blocks
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=0)
    reg = register_tensors(kv, layout)
    chunk = reg.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    region = _native.C.host_region_alloc(NB * bb, hugepage=False, hugepage_bytes=2 << 20, numa_node=-1, populate=True,
                                         touch_threads=16, cuda_register=True, register_chunk_bytes=0, backing_file="")
    host = dict(base=int(region.ptr), layer_stride=shape.kv_dim * chunk, kv_stride=chunk, block_stride=bb,
                num_blocks=NB)
    opts = dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim, chunk_bytes=chunk, max_blocks_per_op=a.blocks,
                h2d=dict(num_ctas=8, tile_bytes=16384, engine=0), d2h=dict(num_ctas=8, tile_bytes=16384, engine=0))
    grp = _native.C.TransferGroup([reg.as_native()], host, opts)
    rng = np.random.default_rng(0)
    rows = []
    for run in a.runs:
        n_runs = a.blocks // run
        starts_g = rng.permutation(NB // run)[:n_runs].astype(np.int64) * run
        starts_c = rng.permutation(NB // run)[:n_runs].astype(np.int64) * run
        g = (starts_g[:, None] + np.arange(run)[None, :]).reshape(-1)
        c = (starts_c[:, None] + np.arange(run)[None, :]).reshape(-1)
        nbytes = len(g) * bb
        for name in ("tma", "ce", "auto"):
            if name == "ce" and run < 4:
                continue                                  # tens of thousands of 32 KiB driver copies: minutes
            row = dict(run_blocks=run, engine=name, bytes=nbytes)
            for h2d in (False, True):
                ms = []
                for i in range(a.iters + 3):
                    r = grp.transfer(g, c, h2d, 0, shape.num_layers, ENG[name])
                    assert r.status == 0, r.status
                    if i >= 3:
                        ms.append(r.gpu_ms)
                row["h2d_gbs" if h2d else "d2h_gbs"] = round(nbytes / float(np.median(ms)) / 1e6, 2)
            rows.append(row)
            print(json.dumps(row), flush=True)
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)
    del grp
    region.free()


if __name__ == "__main__":
    main()
