#!/usr/bin/env python
"""Small, self-terminating driver for profiling the codec copy kernels (lossless bf16 exponent
packing and block-scaled fp8). Moves ``--blocks`` Llama-3-8B-shaped blocks (2 MiB of bf16 each,
N(0,1) values) GPU -> packed host pool -> GPU with the production launch shapes and checks the
round trip (bit-exact for the lossless codec). Sized for an ``ncu`` capture of a handful of
launches: 512 MiB per direction, about 1.5 GiB on the device.
"""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200.models import alloc_paged_cache, get_shape  # noqa: E402
from flexkv_b200.ops import kv_compress as xp  # noqa: E402
from flexkv_b200.ops import kv_quant as q8  # noqa: E402
from flexkv_b200.ops.kv_copy import HostSide, decode_status, new_status  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--codec", default="bf16_xp", choices=["bf16_xp", "fp8_e4m3"])
    ap.add_argument("--blocks", type=int, default=256)
    ap.add_argument("--pool-blocks", type=int, default=512)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--ctas-d2h", type=int, default=48)
    ap.add_argument("--ctas-h2d", type=int, default=32)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    shape = get_shape("llama3-8b")
    kv, layout = alloc_paged_cache(shape, a.pool_blocks, dev, "vllm", fill="normal", seed=1)
    reg = register_tensors(kv, layout)
    elems = reg.chunk_bytes // 2
    L, K = shape.num_layers, shape.kv_dim
    chunk = xp.chunk_slot_bytes(elems) if a.codec == "bf16_xp" else q8.packed_chunk_bytes(elems)
    bb = L * K * chunk
    pool = torch.zeros(a.pool_blocks * bb, dtype=torch.uint8).pin_memory()
    host = HostSide(pool.data_ptr(), K * chunk, chunk, bb, a.pool_blocks)
    table = None
    if a.codec == "bf16_xp":
        table = torch.zeros(xp.size_table_entries(a.pool_blocks, L, K, elems), dtype=torch.int32).pin_memory()
    rng = np.random.default_rng(0)
    status = new_status(dev)
    kv_bytes = a.blocks * L * K * reg.chunk_bytes
    for it in range(a.iters):
        g = rng.permutation(a.pool_blocks)[:a.blocks].astype(np.int64)
        c = rng.permutation(a.pool_blocks)[:a.blocks].astype(np.int64)
        g2 = np.setdiff1d(np.arange(a.pool_blocks), g)[:a.blocks].astype(np.int64)
        for h2d in (False, True):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gb = g2 if h2d else g
            if a.codec == "bf16_xp":
                keep = xp.kv_compress(reg, host, table, gb, c, h2d, num_ctas=a.ctas_h2d if h2d else a.ctas_d2h,
                                      status=status)
            else:
                keep = q8.kv_quant_fp8(reg, host, gb, c, h2d, num_ctas=a.ctas_h2d if h2d else a.ctas_d2h, status=status)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            print(f"iter {it} {a.codec} {'unpack H2D' if h2d else 'pack D2H'}: {ms:.3f} ms  "
                  f"{kv_bytes / ms / 1e6:.2f} GB/s of KV  status={decode_status(status)}")
        gi, g2i = torch.from_numpy(g).to(dev), torch.from_numpy(g2).to(dev)
        if a.codec == "bf16_xp":
            same = all(torch.equal(t[:, gi].view(torch.int16), t[:, g2i].view(torch.int16)) for t in kv)
            used = int(table.view(-1).to(torch.int64).sum()) if it == 0 else 0
            print(f"iter {it} round trip bit-exact: {same}" + (f"  packed/raw = {used / kv_bytes:.4f}" if used else ""))
            assert same
        else:
            err = max(float((t[:, gi].float() - t[:, g2i].float()).abs().max()) for t in kv)
            print(f"iter {it} max abs error after fp8 round trip: {err:.4f}")
    assert decode_status(status) == 0


if __name__ == "__main__":
    main()
