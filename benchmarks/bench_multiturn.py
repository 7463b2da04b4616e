#!/usr/bin/env python
"""Multi-turn serving trace with a byte-exact NVFP4 KV cache and an SSD tier.

Qwen3-32B-shaped cache: 64 layers, 8 KV heads, head_dim 128 stored as NVFP4 (e2m1
nibbles plus one e4m3 scale per 16 elements = 72 bytes per token per head), 16-token
blocks. The packed cache is moved as bytes and must come back bit-identical. Trace:
``--sessions`` sessions x 4 turns, every turn appends 256-2,048 uniform-random tokens;
before a turn the session's history is restored (host pool, else SSD — read straight
into the GPU when --gds is given), after it the whole sequence is offloaded again.
One process per GPU; launch with torchrun for several GPUs (ranks are independent).
"""
import argparse
import json
import os
import sys
import tempfile
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager  # noqa: E402
from flexkv_b200.models import alloc_paged_cache, get_shape, make_model_config  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sessions", type=int, default=512)
    ap.add_argument("--turns", type=int, default=4)
    ap.add_argument("--hbm-gib", type=float, default=64.0)
    ap.add_argument("--host-gib", type=float, default=64.0)
    ap.add_argument("--ssd-gib", type=float, default=128.0)
    ap.add_argument("--ssd-dir", default="")
    ap.add_argument("--gds", action="store_true")
    ap.add_argument("--verify-every", type=int, default=37)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1:
        # --sessions and the pool sizes name the whole box: every rank serves its share, all ranks at once
        a.sessions = max(1, a.sessions // world)
        a.host_gib, a.ssd_gib = a.host_gib / world, a.ssd_gib / world
        if a.out:
            root, ext = os.path.splitext(a.out)
            a.out = f"{root}.rank{rank}{ext}"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    shape = get_shape("qwen3-32b-nvfp4")
    T, bb = shape.tokens_per_block, shape.block_bytes
    NB = int(a.hbm_gib * 2**30) // bb
    ssd_dir = a.ssd_dir or tempfile.mkdtemp(prefix=f"flexkv_ssd_r{rank}_")
    n_ssd = max(2, int(a.ssd_gib * 2**30) // bb)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=int(a.host_gib * 2**30) // bb, enable_ssd=a.ssd_gib > 0,
                      enable_gds=a.gds and a.ssd_gib > 0, num_ssd_blocks=n_ssd, ssd_cache_dir=ssd_dir)
    mgr = KVManager(make_model_config(shape), cfg)
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=a.seed + rank)   # random bytes
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(1800)

    rng = np.random.default_rng(a.seed + 17 * rank)
    hist = [np.zeros(0, dtype=np.int64) for _ in range(a.sessions)]
    ptr = 0
    restored_tok = recomputed_tok = 0
    checked = mismatched = 0
    get_ms, put_ms = [], []
    t_all = time.perf_counter()
    for turn in range(a.turns):
        for s in range(a.sessions):
            new = rng.integers(0, 151936, size=int(rng.integers(256, 2049)), dtype=np.int64)
            tok = np.concatenate([hist[s], new])
            nblk = len(tok) // T
            blocks = ((ptr + np.arange(nblk)) % NB).astype(np.int64)
            ptr = (ptr + nblk) % NB
            slot = np.repeat(blocks, T) * T + np.tile(np.arange(T), nblk)
            verify = a.verify_every and (s % a.verify_every == 0) and turn > 0
            tid, mask = mgr.get_match(tok[:nblk * T])
            hit = int(mask.sum())
            if hit:
                if verify:      # poison the destination so a no-op restore cannot pass
                    idx = torch.from_numpy(blocks[:hit // T]).to(dev)
                    for t in kv[:2]:
                        t[:, idx] = 0
                t0 = time.perf_counter()
                mgr.launch(tid, slot[:hit])
                r = mgr.wait(tid, timeout=300, completely=True)[tid]
                get_ms.append((time.perf_counter() - t0) * 1e3)
                assert r.status.value == "success", r
            restored_tok += hit
            recomputed_tok += nblk * T - hit
            # "prefill" of the tokens that were not restored: fresh random bytes in their blocks
            if nblk * T > hit:
                idx = torch.from_numpy(blocks[hit // T:]).to(dev)
                for t in kv:
                    t[:, idx] = torch.randint(0, 256, t[:, idx].shape, dtype=torch.uint8, device=dev)
            if verify and hit and hasattr(main, "_snap") and s in main._snap:
                want_blocks, want = main._snap[s]
                k = min(len(want_blocks), hit // T)
                got = kv[0][:, torch.from_numpy(blocks[:k]).to(dev)]
                checked += 1
                mismatched += int(not torch.equal(got, want[:, :k]))
            tid, mask = mgr.put_match(tok[:nblk * T])
            if int(mask.sum()):
                t0 = time.perf_counter()
                mgr.launch(tid, slot[mask])
                r = mgr.wait(tid, timeout=300)[tid]
                put_ms.append((time.perf_counter() - t0) * 1e3)
                assert r.status.value == "success", r
            if a.verify_every and s % a.verify_every == 0:
                if not hasattr(main, "_snap"):
                    main._snap = {}
                main._snap[s] = (blocks.copy(), kv[0][:, torch.from_numpy(blocks).to(dev)].clone())
            hist[s] = tok
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_all
    st = mgr.transfer_manager.engine.stats_by_type
    rows = {tt: dict(ops=int(v[0]), blocks=int(v[1]), gib=round(v[2] / 2**30, 2), busy_ms=round(v[3], 1),
                     gbs_while_busy=round(v[2] / v[3] / 1e6, 2) if v[3] else None) for tt, v in st.items()}
    gw = next((w for k, w in (mgr.transfer_manager.engine._workers or {}).items() if k[1].value == "DISK2D"), None)
    out = dict(benchmark="multiturn_nvfp4_ssd", rank=rank, ranks=world, sessions=a.sessions, turns=a.turns, wall_s=round(wall, 2),
               block_bytes=bb, hbm_blocks=NB, host_blocks=cfg.num_cpu_blocks, ssd_blocks=n_ssd,
               restored_tokens=restored_tok, recomputed_tokens=recomputed_tok,
               token_hit_rate=round(restored_tok / max(1, restored_tok + recomputed_tok), 4),
               byte_exact_checks=checked, byte_mismatches=mismatched,
               get_ms_p50=round(float(np.median(get_ms)), 2) if get_ms else None,
               put_ms_p50=round(float(np.median(put_ms)), 2) if put_ms else None,
               gds_direct=bool(gw is not None and gw.direct), per_type=rows)
    print(json.dumps(out))
    if a.out:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    mgr.shutdown()


if __name__ == "__main__":
    main()
