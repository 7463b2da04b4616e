#!/usr/bin/env python
"""Small, self-terminating driver for profiling the paged KV copy kernel.

Moves ``--blocks`` Llama-3-8B-shaped blocks (2 MiB each) GPU->host and back a few
times with the production launch shape; sized so that an ``ncu`` capture of a
handful of launches ends by itself (a few hundred MiB on the device, inputs
larger than L2). Prints the CUDA-event time of every launch.
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200.models import alloc_paged_cache, get_shape  # noqa: E402
from flexkv_b200.ops.kv_copy import HostSide, decode_status, kv_copy, new_status  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--blocks", type=int, default=256)      # 512 MiB per direction
    ap.add_argument("--pool-blocks", type=int, default=512)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--ctas", type=int, default=8)
    ap.add_argument("--tile-bytes", type=int, default=16384)
    ap.add_argument("--engine", type=int, default=0)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    shape = get_shape(a.model)
    kv, layout = alloc_paged_cache(shape, a.pool_blocks, dev, "vllm", fill="normal", seed=1)
    reg = register_tensors(kv, layout)
    chunk = reg.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    pool = torch.empty(a.pool_blocks * bb, dtype=torch.uint8).pin_memory()
    host = HostSide(pool.data_ptr(), shape.kv_dim * chunk, chunk, bb, a.pool_blocks)
    rng = np.random.default_rng(0)
    status = new_status(dev)
    for it in range(a.iters):
        g = rng.permutation(a.pool_blocks)[:a.blocks].astype(np.int64)
        c = rng.permutation(a.pool_blocks)[:a.blocks].astype(np.int64)
        for h2d in (False, True):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            keep = kv_copy(reg, host, g, c, h2d=h2d, num_ctas=a.ctas, tile_bytes=a.tile_bytes, engine=a.engine,
                           status=status)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            print(f"iter {it} {'H2D' if h2d else 'D2H'}: {ms:.3f} ms  {a.blocks * bb / ms / 1e6:.2f} GB/s "
                  f"status={decode_status(status)}")
    assert decode_status(status) == 0


if __name__ == "__main__":
    main()
