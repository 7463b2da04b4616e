#!/usr/bin/env python
"""One batch through the public API: put a batch of sequences, then get it back.

Same flags and config file format as the reference's script of this name
(benchmarks/benchmark_single_batch.py:27-160): model geometry and tier sizes come from a flat
YAML/JSON file; ``--cache-ratio`` is the share of each sequence that is offloaded before the get;
``--clear-cpu-cache`` drops the host tier between put and get so that the get comes from SSD.
Bandwidth = tokens moved x bytes per token / elapsed, as the reference computes it.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.common.config import (ModelConfig, UserConfig, parse_dtype,  # noqa: E402
                                       update_default_config_from_user_config)
from flexkv_b200.models import KVShape, alloc_paged_cache  # noqa: E402


def load(path: str):
    with open(path) as f:
        if path.endswith((".yml", ".yaml")):
            import yaml
            raw = yaml.safe_load(f)
        else:
            raw = json.load(f)
    m = ModelConfig(num_layers=raw["num_layers"], num_kv_heads=raw["num_kv_heads"], head_size=raw["head_size"],
                    dtype=parse_dtype(raw.get("dtype", "bfloat16")), kv_dim=raw.get("kv_dim", 2),
                    use_mla=bool(raw.get("use_mla", False)), tp_size=raw.get("tp_size", 1), dp_size=raw.get("dp_size", 1))
    c = CacheConfig(tokens_per_block=raw.get("tokens_per_block", 16))
    known = {f for f in UserConfig.__dataclass_fields__}
    u = UserConfig(**{k: v for k, v in raw.items() if k in known})
    return m, c, u


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, default=os.path.join(os.path.dirname(__file__), "example_config.yml"))
    ap.add_argument("--num-layers", type=int, default=-1)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--sequence-length", type=int, default=1024)
    ap.add_argument("--cache-ratio", type=float, default=1)
    ap.add_argument("--clear-cpu-cache", action="store_true")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    model, cache, user = load(a.config)
    if a.num_layers > 0:
        model.num_layers = a.num_layers
    update_default_config_from_user_config(model, cache, user)
    T = cache.tokens_per_block
    shape = KVShape("bench", model.num_layers, model.num_kv_heads, model.head_size, dtype=model.dtype,
                    use_mla=model.use_mla, tokens_per_block=T)
    blocks_per_seq = a.sequence_length // T
    nb = a.batch_size * blocks_per_seq
    mgr = KVManager(model, cache, require_gpu=True, in_process=True)
    kv, layout = alloc_paged_cache(shape, max(nb, 2), a.device if a.device == "cpu" else torch.device(a.device), "vllm",
                                   tp_size=model.tp_size, fill="normal")
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(600)
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 100000, size=blocks_per_seq * T, dtype=np.int64) for _ in range(a.batch_size)]
    slot = [np.arange(i * blocks_per_seq * T, (i + 1) * blocks_per_seq * T, dtype=np.int64) for i in range(a.batch_size)]
    keep = int(blocks_per_seq * a.cache_ratio) * T
    token_bytes = model.token_size_in_bytes
    t0 = time.perf_counter()
    tids = [mgr.put_async(s[:keep], m[:keep]) for s, m in zip(seqs, slot)] if keep else []
    res = mgr.wait(tids, completely=True) if tids else {}
    put_s = time.perf_counter() - t0
    put_tokens = sum(int(r.return_mask.sum()) for r in res.values())
    if a.clear_cpu_cache:
        mgr._clear_cpu_cache()
    t0 = time.perf_counter()
    tids, masks = [], []
    for s in seqs:
        tid, mask = mgr.get_match(s)
        tids.append(tid); masks.append(mask)
    mgr.launch(tids, [m[mk] for m, mk in zip(slot, masks)], as_batch=True)
    mgr.wait(tids)
    get_s = time.perf_counter() - t0
    get_tokens = sum(int(m.sum()) for m in masks)
    print(json.dumps(dict(batch_size=a.batch_size, sequence_length=a.sequence_length, cache_ratio=a.cache_ratio,
                          put_tokens=put_tokens, put_ms=round(put_s * 1e3, 2),
                          put_gbs=round(put_tokens * token_bytes / max(put_s, 1e-9) / 1e9, 2),
                          get_tokens=get_tokens, get_ms=round(get_s * 1e3, 2),
                          get_gbs=round(get_tokens * token_bytes / max(get_s, 1e-9) / 1e9, 2))))
    mgr.shutdown()


if __name__ == "__main__":
    main()
