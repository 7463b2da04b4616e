#!/usr/bin/env python
"""DeepSeek-V3-shaped MLA cache on N data-parallel ranks of one box (one process drives
every GPU): 61 layers, a 576-wide latent per token (512 kv_lora + 64 rope), bf16,
64-token blocks. Offload packs to fp8 e4m3 with one fp32 scale per 128 values (or stays
raw / lossless with --codec). A share of the requests (default 30 %) reuses a prefix that
currently sits in ANOTHER rank's GPU blocks; those blocks are pulled over NVLink instead
of being read from host memory. Trace: 256 requests of 4K-32K tokens, 32 shared prefixes,
all ids and values seeded.
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
from flexkv_b200.models import alloc_paged_cache, get_shape, make_model_config  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=torch.cuda.device_count())
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--gpu-blocks", type=int, default=3072)
    ap.add_argument("--host-gib", type=float, default=48.0)
    ap.add_argument("--codec", default="fp8_e4m3", choices=["none", "bf16_xp", "fp8_e4m3"])
    ap.add_argument("--peer-share", type=float, default=0.30)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="")
    ap.add_argument("--concurrent", action="store_true",
                    help="drive every rank from its own thread (all links busy at once) instead of one request at a time")
    a = ap.parse_args()
    N = a.gpus
    shape = get_shape("deepseek-v3")
    T = shape.tokens_per_block
    bb = shape.block_bytes
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=int(a.host_gib * 2**30) // bb, enable_p2p_gpu=N > 1,
                      offload_quant="fp8_e4m3" if a.codec == "fp8_e4m3" else "none",
                      enable_compression=a.codec == "bf16_xp")
    mgr = KVManager(make_model_config(shape, dp_size=N), cfg, in_process=True)
    caches = []
    for d in range(N):
        kv, layout = alloc_paged_cache(shape, a.gpu_blocks, torch.device("cuda", d), "vllm", fill="normal",
                                       seed=a.seed + d)
        mgr.register_gpu_tensors(kv, layout, dp_client_id=d)
        caches.append(kv)
    mgr.start()
    mgr.wait_ready(900)
    eng = mgr.kv_task_engine

    rng = np.random.default_rng(a.seed)
    prefixes = [rng.integers(0, 129280, size=int(rng.integers(2048, 16385)) // T * T, dtype=np.int64) for _ in range(32)]
    resident = {}          # prefix id -> (rank, gpu blocks) currently published
    free_ptr = [0] * N     # ring allocation of GPU blocks per rank

    def take_blocks(rank, n):
        s = free_ptr[rank]
        ids = (np.arange(s, s + n) % a.gpu_blocks).astype(np.int64)
        free_ptr[rank] = (s + n) % a.gpu_blocks
        # blocks about to be reused are withdrawn from the peer directory first
        mgr.withdraw_gpu_blocks(ids, dp_client_id=rank)
        for pid, (r, blk) in list(resident.items()):
            if r == rank and np.intersect1d(blk, ids).size:
                del resident[pid]
        return ids

    import threading
    state_lock = threading.Lock()          # guards `resident` and the block rings
    counts = {"peer": 0, "host": 0}

    def serve(i: int) -> None:
        """request i: restore whatever prefix is cached (a peer's HBM first, then host), offload the rest"""
        rank = i % N
        r_i = np.random.default_rng([a.seed, i])
        n = int(r_i.integers(4096, 32769)) // T * T
        with state_lock:
            others = [p for p, (r, _) in resident.items() if r != rank]
            use_peer = N > 1 and r_i.random() < a.peer_share and bool(others)
            pid = int(r_i.choice(others)) if use_peer else int(r_i.integers(32))
            nblk = n // T
            blocks = take_blocks(rank, nblk)
        pre = prefixes[pid][:n]
        tok = np.concatenate([pre, r_i.integers(0, 129280, size=n - len(pre), dtype=np.int64)])
        slot = np.repeat(blocks, T) * T + np.tile(np.arange(T), nblk)
        tid, mask = eng.get_match(tok, None, rank)
        hit = int(mask.sum())
        if hit:
            eng.launch_tasks([tid], [slot[:hit]])
            r = eng.wait([tid], timeout=300)[tid]
            assert r.status.value == "success", r
            with state_lock:
                counts["peer" if use_peer else "host"] += 1
        tid, mask = eng.put_match(tok, None, rank)
        if int(mask.sum()):
            eng.launch_tasks([tid], [slot[mask]])
            r = eng.wait([tid], timeout=300, completely=True)[tid]
            assert r.status.value == "success", r
        # the request's prefix now lives in this rank's GPU blocks
        k = len(pre) // T
        mgr.publish_gpu_blocks(tok[:k * T], slot[:k * T], dp_client_id=rank)
        with state_lock:
            resident[pid] = (rank, blocks[:k])

    t0 = time.perf_counter()
    if a.concurrent and N > 1:
        # every rank is driven by its own thread, as N engine processes would: all PCIe links and the
        # NVLink pulls are busy at the same time
        errs = []

        def rank_loop(rank: int) -> None:
            try:
                for i in range(rank, a.requests, N):
                    serve(i)
            except Exception as e:  # noqa: BLE001
                errs.append(f"rank {rank}: {type(e).__name__}: {e}")
        ths = [threading.Thread(target=rank_loop, args=(r,)) for r in range(N)]
        for th in ths:
            th.start()
        for th in ths:
            th.join()
        if errs:
            raise RuntimeError("; ".join(errs[:3]))
    else:
        for i in range(a.requests):
            serve(i)
    peer_req, host_req = counts["peer"], counts["host"]
    for d in range(N):
        torch.cuda.synchronize(d)
    wall = time.perf_counter() - t0
    st = mgr.transfer_manager.engine.stats_by_type
    rows = {}
    for tt, (ops, blocks, nbytes, ms) in st.items():
        rows[tt] = dict(ops=int(ops), blocks=int(blocks), gib=round(nbytes / 2**30, 2),
                        busy_ms=round(ms, 1), gbs_while_busy=round(nbytes / ms / 1e6, 2) if ms else None)
    out = dict(benchmark="mla_dp_prefix_reuse", gpus=N, codec=a.codec, requests=a.requests, wall_s=round(wall, 2),
               ranks_driven="concurrently, one thread per rank" if a.concurrent and N > 1 else "one request at a time",
               requests_served_from_peer_gpu=peer_req, requests_served_from_host=host_req, per_type=rows,
               peer_directory=eng.cache_engine.peer_directory.stats if eng.cache_engine.peer_directory else None)
    print(json.dumps(out))
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    mgr.shutdown()


if __name__ == "__main__":
    main()
