#!/usr/bin/env python
"""Smallest complete use of the manager: offload a prompt's KV, drop the host copy, restore it from SSD.

    python examples/standalone_roundtrip.py              # cuda:0 when there is one, else the CPU data plane
    python examples/standalone_roundtrip.py --device cpu
"""
import argparse
import os
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape, make_model_config  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tokens", type=int, default=1024)
    a = ap.parse_args()
    shape = get_shape("llama3-8b")                       # 32 layers x 8 KV heads x 128, bf16, 16-token pages
    T = shape.tokens_per_block
    n = a.tokens // T
    with tempfile.TemporaryDirectory() as ssd_dir:
        mgr = KVManager(make_model_config(shape),
                        CacheConfig(tokens_per_block=T, num_cpu_blocks=4 * n, enable_ssd=True,
                                    num_ssd_blocks=8 * n, ssd_cache_dir=ssd_dir), require_gpu=True)
        dev = a.device if a.device == "cpu" else torch.device(a.device)
        kv, layout = alloc_paged_cache(shape, 4 * n, dev, "vllm", fill="normal", seed=0)   # the engine's paged cache
        mgr.register_gpu_tensors(kv, layout)
        mgr.start()
        mgr.wait_ready(120)
        try:
            tokens = np.arange(a.tokens, dtype=np.int64)
            src = np.arange(n, dtype=np.int64)                              # pages that hold the prompt's KV
            slots = np.repeat(src, T) * T + np.tile(np.arange(T), n)
            tid = mgr.put_async(tokens, slots)                              # GPU -> host -> SSD (write-through)
            assert mgr.wait(tid, completely=True)[tid].ok
            want = [t[:, src].clone() for t in kv]
            mgr._clear_cpu_cache()                                          # noqa: SLF001 - force the SSD path
            tid, mask = mgr.get_match(tokens)                               # what is cached, on any tier
            dst = np.arange(2 * n, 3 * n, dtype=np.int64)
            mgr.launch(tid, (np.repeat(dst, T) * T + np.tile(np.arange(T), n))[mask])
            rsp = mgr.wait(tid)[tid]
            same = all(torch.equal(t[:, dst], w) for t, w in zip(kv, want))
            print(f"restored {rsp.num_tokens()} of {a.tokens} tokens from SSD on {a.device}: "
                  f"status={rsp.status.value}, bytes identical={same}")
            return 0 if rsp.ok and same else 1
        finally:
            mgr.shutdown()


if __name__ == "__main__":
    sys.exit(main())
