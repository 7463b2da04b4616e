#!/usr/bin/env python
"""NVLink paths against their baselines, timed with CUDA events (max over ranks).

``python benchmarks/bench_nvlink.py --mode pull``   (one process, >= 2 GPUs)
    Prefix pull of scattered blocks out of a peer's paged cache (DeepSeek-V3 MLA latent
    blocks: 61 layers, 64 tokens x 576 x bf16 = 72 KiB per layer and block) with the pull
    kernel, against one peer memcpy per (layer, block) chunk issued from the host, and
    against a single contiguous peer memcpy of the same byte count (link roofline).

``torchrun --nproc-per-node N benchmarks/bench_nvlink.py --mode fanout``
    Shared-KV restore at TP=N: rank 0 reads the host blocks once and multimem-stores them
    to every rank (one PCIe read), against every rank restoring the same blocks itself
    (N PCIe reads of the same bytes, the reference's way).
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.common.storage import KVCacheLayout, KVCacheLayoutType  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402

L, T, D = 61, 64, 576


def mode_pull(a):
    n_gpu = torch.cuda.device_count()
    if n_gpu < 2:
        print(json.dumps({"mode": "pull", "skipped": "needs 2 GPUs"}))
        return []
    NB, n = a.gpu_blocks, a.blocks
    regs, caches = [], []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        g = torch.Generator(device=dev).manual_seed(d + 1)
        kv = [torch.randn(NB, T, D, dtype=torch.bfloat16, device=dev, generator=g) for _ in range(L)]
        lay = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, NB, T, 1, D, is_mla=True)
        regs.append(register_tensors(kv, lay))
        caches.append(kv)
    chunk = regs[0].chunk_bytes
    total = n * L * chunk
    rng = np.random.default_rng(0)
    src = rng.permutation(NB)[:n].astype(np.int64)
    dst = rng.permutation(NB)[:n].astype(np.int64)
    rows = []
    for ctas, tile in [(c, t) for t in a.tile_bytes for c in a.ctas]:
        copier = _native.C.PeerCopier([r.as_native() for r in regs], L, 1, chunk, num_ctas=ctas, tile_bytes=tile,
                                      engine=0, max_blocks_per_op=max(4096, n))
        if not copier.can_access(0, 1):
            print(json.dumps({"mode": "pull", "skipped": "no peer access between GPU 0 and 1"}))
            return rows
        ms = []
        for i in range(a.iters + 3):
            r = copier.pull(0, 1, dst, src, 0, L)
            assert r.status == 0, r.status
            if i >= 3:
                ms.append(r.gpu_ms)
        t = float(np.median(ms))
        rows.append(dict(mode="pull", path="pull_kernel", ctas=ctas, tile_bytes=tile, blocks=n, bytes=total, ms=round(t, 3),
                         gbs=round(total / t / 1e6, 1)))
        print(json.dumps(rows[-1]), flush=True)
        del copier
    # byte check of the last pull
    for l in (0, L - 1):
        assert torch.equal(caches[0][l][torch.from_numpy(dst).cuda(0)].cpu(), caches[1][l][torch.from_numpy(src).cuda(1)].cpu())
    # baseline 1: one peer copy per (layer, block) chunk
    torch.cuda.set_device(0)
    s = torch.cuda.Stream(device=0)
    ms = []
    nb_base = min(n, a.baseline_blocks)
    for i in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s):
            e0.record()
            for l in range(L):
                dl, sl = caches[0][l], caches[1][l]
                for k in range(nb_base):
                    dl[int(dst[k])].copy_(sl[int(src[k])], non_blocking=True)
            e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = float(np.median(ms))
    b = nb_base * L * chunk
    rows.append(dict(mode="pull", path="memcpy_peer_per_chunk", blocks=nb_base, bytes=b, ms=round(t, 3),
                     gbs=round(b / t / 1e6, 1)))
    print(json.dumps(rows[-1]), flush=True)
    # baseline 2: one contiguous peer copy of the same size (what the link gives)
    flat0 = torch.empty(total, dtype=torch.uint8, device="cuda:0")
    flat1 = torch.empty(total, dtype=torch.uint8, device="cuda:1")
    ms = []
    for i in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s):
            e0.record()
            flat0.copy_(flat1, non_blocking=True)
            e1.record()
        e1.synchronize()
        if i >= 2:
            ms.append(e0.elapsed_time(e1))
    t = float(np.median(ms))
    rows.append(dict(mode="pull", path="memcpy_peer_contiguous", bytes=total, ms=round(t, 3),
                     gbs=round(total / t / 1e6, 1)))
    print(json.dumps(rows[-1]), flush=True)
    return rows


def mode_fanout(a):
    import torch.distributed as dist
    from flexkv_b200.ops.kv_copy import HostSide, decode_status, kv_copy, new_status
    from flexkv_b200.parallel.nvls import alloc_symmetric_kv, fanout_restore, wait_flag
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rows = []
    try:
        NB, n = a.gpu_blocks, a.blocks
        per_layer = NB * T * D * 2
        try:
            if a.segment_gib > 0:
                # layers in symmetric segments of at most --segment-gib, one multicast object each
                from flexkv_b200.parallel.nvls import alloc_symmetric_kv_layers
                sym = alloc_symmetric_kv_layers(L, per_layer, dev, segment_bytes=int(a.segment_gib * 2**30))
                kv = [sym.layer_tensor(l, (NB, T, D), torch.bfloat16) for l in range(L)]
            else:
                sym = alloc_symmetric_kv(L * per_layer, dev)
                kv = [sym.carve(l * per_layer, (NB, T, D), torch.bfloat16) for l in range(L)]
        except RuntimeError as e:
            if rank == 0:
                print(json.dumps({"mode": "fanout", "skipped": str(e)}))
            return rows
        lay = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, NB, T, 1, D, is_mla=True)
        reg = register_tensors(kv, lay)
        chunk = reg.chunk_bytes
        g = torch.Generator().manual_seed(5)      # same host bytes on every rank
        pool = torch.randint(0, 256, (n, L, 1, chunk), dtype=torch.uint8, generator=g).pin_memory()
        host = HostSide(pool.data_ptr(), chunk, chunk, L * chunk, n)
        rng = np.random.default_rng(1)
        gpu_blocks = rng.permutation(NB)[:n].astype(np.int64)
        cpu_blocks = np.arange(n, dtype=np.int64)
        total = n * L * chunk
        status = new_status(dev)
        scratch = torch.zeros(1, dtype=torch.int32, device=dev)

        def timed_max(ms_local):
            t = torch.tensor([ms_local], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        # every rank restores for itself
        ms = []
        for i in range(a.iters + 3):
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            keep = kv_copy(reg, host, gpu_blocks, cpu_blocks, h2d=True, num_ctas=8, tile_bytes=16384, status=status)
            e1.record()
            torch.cuda.synchronize()
            t = timed_max(e0.elapsed_time(e1))
            if i >= 3:
                ms.append(t)
        errors = []
        if decode_status(status) != 0:
            errors.append(f"copy status {decode_status(status)}")
        t_ind = float(np.median(ms))
        gidx = torch.from_numpy(gpu_blocks).to(dev)
        check_layers = list(range(L))     # every layer: a partial multicast mapping shows up as a suffix of bad layers
        want = {l: kv[l][gidx].clone() for l in check_layers}

        def compare():
            """(mismatching blocks per checked layer, description of the first mismatch)"""
            bad, first = {}, ""
            for l in check_layers:
                got = kv[l][gidx]
                neq = (got.view(torch.int16) != want[l].view(torch.int16)).reshape(n, -1)
                per_block = neq.any(dim=1)
                k = int(per_block.sum())
                if k:
                    bad[l] = k
                    if not first:
                        b = int(per_block.nonzero()[0])
                        off = int(neq[b].nonzero()[0])
                        zero = bool((got[b].view(torch.int16) == 0).all())
                        first = (f"layer {l} pair {b} (gpu block {int(gpu_blocks[b])}) first differing element {off} "
                                 f"of {neq.shape[1]}, {int(neq[b].sum())} elements differ, block all zero: {zero}")
            return bad, first
        # library baseline: rank 0 restores for itself, gathers the restored blocks, NCCL broadcasts them and
        # every other rank scatters them into its cache (one PCIe read too, but three passes over HBM and no overlap)
        ms = []
        for i in range(a.iters + 3):
            torch.cuda.synchronize(); dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if rank == 0:
                keep = kv_copy(reg, host, gpu_blocks, cpu_blocks, h2d=True, num_ctas=8, tile_bytes=16384, status=status)
                stage = torch.stack([kv[l][gidx] for l in range(L)])
            else:
                stage = torch.empty((L, n, T, D), dtype=torch.bfloat16, device=dev)
            dist.broadcast(stage, src=0)
            if rank != 0:
                for l in range(L):
                    kv[l][gidx] = stage[l]
            e1.record()
            torch.cuda.synchronize()
            t = timed_max(e0.elapsed_time(e1))
            if i >= 3:
                ms.append(t)
            del stage
        t_nccl = float(np.median(ms))
        bad, first = compare()
        if bad:
            errors.append(f"NCCL baseline: bytes differ on rank {rank}: {bad}; {first}")
        # one reader, NVSwitch multicast
        for ctas in a.ctas:
            ms = []
            for i in range(a.iters + 3):
                epoch = 100 * ctas + i + 1
                if i == 0:
                    for t_ in kv:
                        t_.zero_()
                torch.cuda.synchronize(); dist.barrier()
                t0 = time.perf_counter()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if rank == 0:
                    e0.record()
                    keep = fanout_restore(sym, reg, host, gpu_blocks, cpu_blocks, epoch, scratch, status, num_ctas=ctas)
                    e1.record()
                ok = wait_flag(sym, epoch, timeout_s=20.0)
                wall = (time.perf_counter() - t0) * 1e3
                torch.cuda.synchronize()
                if not ok:
                    errors.append("completion flag never arrived")
                t = timed_max(e0.elapsed_time(e1) if rank == 0 else 0.0)
                w = timed_max(wall)
                if i >= 3:
                    ms.append((t, w))
            # every rank walks the same collective sequence whatever it found: a rank must not leave
            # while its memory is bound to the multicast object
            bad, first = compare()
            if bad:
                errors.append(f"bytes differ on rank {rank}: blocks per layer {bad}; {first}")
                if rank <= 1 or rank == world - 1:
                    print(json.dumps({"mode": "fanout", "rank": rank, "ctas": ctas, "mismatch": errors[-1]}), flush=True)
            bad = torch.tensor([len(errors)], dtype=torch.float64, device=dev)
            dist.all_reduce(bad, op=dist.ReduceOp.SUM)
            t_fan = float(np.median([m[0] for m in ms]))
            w_fan = float(np.median([m[1] for m in ms]))
            if rank == 0:
                rows.append(dict(mode="fanout", ranks=world, ctas=ctas, bytes_per_rank=total,
                                 symmetric_segment_gib=a.segment_gib, cache_gib=round(L * per_layer / 2**30, 2),
                                 independent_h2d_ms=round(t_ind, 3), h2d_then_nccl_broadcast_ms=round(t_nccl, 3),
                                 fanout_kernel_ms=round(t_fan, 3),
                                 fanout_until_flag_seen_ms_host_clock=round(w_fan, 3),
                                 host_bytes_read_independent=total * world, host_bytes_read_fanout=total,
                                 delivered_gbs_fanout=round(total * world / t_fan / 1e6, 1),
                                 delivered_gbs_independent=round(total * world / t_ind / 1e6, 1),
                                 errors_over_ranks=int(bad.item()), rank0_errors=errors[:3]))
                print(json.dumps(rows[-1]), flush=True)
            dist.barrier()
        return rows
    finally:
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="pull", choices=["pull", "fanout"])
    ap.add_argument("--segment-gib", type=float, default=2.0,
                    help="fan-out: size of one symmetric segment (0 = the whole cache in one allocation)")
    ap.add_argument("--blocks", type=int, default=256)
    ap.add_argument("--gpu-blocks", type=int, default=1024)
    ap.add_argument("--baseline-blocks", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, nargs="+", default=[8, 32, 64])
    ap.add_argument("--tile-bytes", type=int, nargs="+", default=[16384], help="pull: tile sizes of the copy kernel")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rows = mode_pull(a) if a.mode == "pull" else mode_fanout(a)
    if a.out and rows:
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
