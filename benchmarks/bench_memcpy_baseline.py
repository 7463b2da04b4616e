#!/usr/bin/env python
"""Copy-engine ceiling of the box: every rank copies one contiguous pinned buffer to and from
its GPU at the same time (`cudaMemcpyAsync` through torch), CUDA events, max over ranks.
This is what the PCIe links and the host memory system give N GPUs at once, the denominator
for the multi-GPU numbers of bench.py. Launch with torchrun (one rank per GPU) or plain for one GPU.
"""
import argparse
import json
import os

import numpy as np
import torch


def _write_combined_host_tensor(n: int) -> torch.Tensor:
    """n bytes from cudaHostAlloc(portable | write-combined), wrapped as a tensor; never freed (benchmark)."""
    import ctypes
    import glob
    import site
    libs = []
    for root in site.getsitepackages() + [os.path.dirname(torch.__file__)]:
        libs += glob.glob(os.path.join(root, "nvidia", "cuda_runtime", "lib", "libcudart.so*"))
        libs += glob.glob(os.path.join(root, "lib", "libcudart*.so*"))
    rt = ctypes.CDLL(libs[0] if libs else "libcudart.so")
    ptr = ctypes.c_void_p()
    rc = rt.cudaHostAlloc(ctypes.byref(ptr), ctypes.c_size_t(n), ctypes.c_uint(0x01 | 0x04))
    if rc != 0 or not ptr.value:
        raise RuntimeError(f"cudaHostAlloc(write-combined) failed with error {rc}")
    buf = (ctypes.c_uint8 * n).from_address(ptr.value)
    t = torch.frombuffer(buf, dtype=torch.uint8)
    t._keep = buf
    return t


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gib", type=float, default=4.0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--per-block-kib", type=int, nargs="*", default=[],
                    help="also copy the same bytes as one cudaMemcpyAsync per block of this size, blocks at random "
                         "positions on both sides (what a copy-engine path without staging would issue)")
    ap.add_argument("--streams", type=int, nargs="*", default=[1, 4])
    ap.add_argument("--host-alloc", default="pinned", choices=["pinned", "wc"],
                    help="wc: the host buffer comes from cudaHostAlloc with the write-combined flag (the CPU does "
                         "not cache it, so device writes need no snoop of CPU caches)")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    n = int(a.gib * 2**30)
    if a.host_alloc == "wc":
        host = _write_combined_host_tensor(n)
    else:
        host = torch.empty(n, dtype=torch.uint8).pin_memory()
        host.fill_(1)
    gpu = torch.empty(n, dtype=torch.uint8, device=dev)
    out = {}
    for name, (dst, src) in (("d2h", (host, gpu)), ("h2d", (gpu, host))):
        ms = []
        for i in range(a.iters + 3):
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dst.copy_(src, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            if dist is not None:
                dist.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            if i >= 3:
                ms.append(float(t.item()))
        out[name + "_gbs_per_gpu"] = round(n / float(np.median(ms)) / 1e6, 2)
    # one driver copy per block, blocks scattered on both sides
    for kib in a.per_block_kib:
        blk = kib * 1024
        nb = n // blk
        rng = np.random.default_rng(7)
        pg, ph = rng.permutation(nb).tolist(), rng.permutation(nb).tolist()
        g2d, h2d_ = gpu[:nb * blk].view(nb, blk), host[:nb * blk].view(nb, blk)
        for ns in a.streams:
            streams = [torch.cuda.Stream() for _ in range(ns)]
            for name, (dst, src, pd, ps) in (("d2h", (h2d_, g2d, ph, pg)), ("h2d", (g2d, h2d_, pg, ph))):
                ms = []
                for i in range(3):
                    torch.cuda.synchronize()
                    e0 = torch.cuda.Event(enable_timing=True)
                    ends = [torch.cuda.Event(enable_timing=True) for _ in streams]
                    e0.record()
                    for k, st in enumerate(streams):
                        st.wait_event(e0)
                        with torch.cuda.stream(st):
                            for j in range(k, nb, ns):
                                dst[pd[j]].copy_(src[ps[j]], non_blocking=True)
                            ends[k].record(st)
                    torch.cuda.synchronize()
                    if i >= 1:
                        ms.append(max(e0.elapsed_time(e) for e in ends))
                out[f"{name}_per_block_{kib}KiB_{ns}streams_gbs"] = round(nb * blk / float(np.median(ms)) / 1e6, 2)
    # both directions at once (a put on one stream, a get on another)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    host2 = torch.empty(n, dtype=torch.uint8).pin_memory()
    gpu2 = torch.empty(n, dtype=torch.uint8, device=dev)
    ms = []
    for i in range(a.iters + 3):
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        s1.wait_event(e0); s2.wait_event(e0)
        with torch.cuda.stream(s1):
            host.copy_(gpu, non_blocking=True); e1.record(s1)
        with torch.cuda.stream(s2):
            gpu2.copy_(host2, non_blocking=True); e2.record(s2)
        torch.cuda.synchronize()
        t = torch.tensor([max(e0.elapsed_time(e1), e0.elapsed_time(e2))], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        if i >= 3:
            ms.append(float(t.item()))
    out["bidirectional_gbs_per_gpu_sum"] = round(2 * n / float(np.median(ms)) / 1e6, 2)
    if rank == 0:
        print(json.dumps(dict(benchmark="memcpy_baseline", gpus=world, gib_per_copy=a.gib, host_alloc=a.host_alloc,
                         host_is_pinned=bool(host.is_pinned()), **out)))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
