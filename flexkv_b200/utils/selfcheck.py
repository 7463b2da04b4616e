"""Byte-exact self checks of the data plane on real GPUs, small enough to run after a benchmark.

Each function builds its own small caches, moves data through the native path under test and
compares every byte with a PyTorch gather of the same blocks. They return ``True``/``False`` (or
raise on a launch error); ``bench.py`` prints their results under ``verified`` and the GPU tests
assert on them, so the multi-GPU paths are proven wherever two or more GPUs are visible.

The scenarios mirror the reference's data-plane correctness suite
(``tests/test_kv_transfer_correctness.py:515-520,604-610`` TP thread group with MHA slices and the
shared-KV write modes, ``:1320-1327`` layerwise restore) and add the NVLink peer pull, which the
reference does not have.
"""
from __future__ import annotations

import os
import struct
from typing import Dict, Sequence

import numpy as np
import torch

from .. import CacheConfig, KVManager, _native
from ..common.transfer import TransferType, WorkerKey
from ..models import KVShape, alloc_paged_cache, make_model_config
from ..storage.gpu_layout import register_tensors

SHARED_KV_MODES = ("sharded", "all_write", "rank0_only", "layer_parallel", "rank_rotate")
last_failure = ""      # where the most recent check that returned False went wrong


def _fail(why: str) -> bool:
    global last_failure
    last_failure = why
    return False


def slots_of(blocks, tokens_per_block: int) -> np.ndarray:
    b = np.asarray(blocks, dtype=np.int64)
    return np.repeat(b, tokens_per_block) * tokens_per_block + np.tile(np.arange(tokens_per_block), len(b))


def manager_roundtrip(mgr: KVManager, kv: Sequence[torch.Tensor], gpu_blocks: int, tokens_per_block: int,
                      n_blocks: int = 64, seed: int = 4321, vocab: int = 128256, layers=None) -> bool:
    """put -> get of ``n_blocks`` fresh blocks through the public API into *different* GPU blocks of a
    vLLM-layout cache, then compare source and destination pages of the given layers."""
    T = tokens_per_block
    r = np.random.default_rng(seed)
    tok = r.integers(0, vocab, size=n_blocks * T, dtype=np.int64)
    ids = r.permutation(gpu_blocks)[:2 * n_blocks].astype(np.int64)
    src, dst = ids[:n_blocks], ids[n_blocks:]
    tid = mgr.put_async(tok, slots_of(src, T))
    if mgr.wait(tid, timeout=120, completely=True)[tid].status.value != "success":
        return False
    tid, mask = mgr.get_match(tok)
    if int(mask.sum()) != n_blocks * T:
        return False
    mgr.launch(tid, slots_of(dst, T))
    if mgr.wait(tid, timeout=120)[tid].status.value != "success":
        return False
    torch.cuda.synchronize(kv[0].device)
    a = torch.from_numpy(src).to(kv[0].device)
    b = torch.from_numpy(dst).to(kv[0].device)
    L = len(kv)
    for l in (layers if layers is not None else sorted({0, L // 2, L - 1})):
        t = kv[l]
        same = torch.equal(t[:, a], t[:, b]) if t.dim() >= 4 and t.shape[0] == 2 else torch.equal(t[a], t[b])
        if not same:
            return False
    return True


def tp_group_two_gpus(mode: str = "mha", devices=(0, 1)) -> bool:
    """TP transfer group on two GPUs: offload into one shared host block, restore into other pages.
    ``mode`` = "mha" (each rank owns its head slice) or one of the shared-KV write modes."""
    C = _native.C
    mla = mode != "mha"
    shape = KVShape("t", 4, 1 if mla else 4, 128 if mla else 32, use_mla=mla, tokens_per_block=16)
    caches, regs = [], []
    for i, d in enumerate(devices):
        kv, layout = alloc_paged_cache(shape, 48, torch.device("cuda", d), "vllm", tp_size=1 if mla else 2,
                                       fill="normal", seed=40 if mla else 40 + i)
        caches.append(kv)
        regs.append(register_tensors(kv, layout))
    chunk = regs[0].chunk_bytes
    slices = 1 if mla else 2
    K = shape.kv_dim
    block_bytes = slices * 4 * K * chunk
    pool = torch.zeros(48, block_bytes, dtype=torch.uint8).pin_memory()
    host = dict(base=pool.data_ptr(), layer_stride=K * chunk, kv_stride=chunk, block_stride=block_bytes, num_blocks=48)
    opts = dict(num_layers=4, kv_dim=K, chunk_bytes=chunk, cpu_tp_stride=block_bytes // slices, shared_kv=mla,
                shared_mode=mode if mla else "sharded", max_blocks_per_op=64)
    grp = C.TransferGroup([r.as_native() for r in regs], host, opts)
    g = np.array([3, 40, 11, 7, 25], dtype=np.int64)
    c = np.array([9, 0, 47, 2, 30], dtype=np.int64)
    st = grp.transfer(g, c, False, 0, 4).status
    if st != 0:
        return _fail(f"{mode}: offload status {st}")
    ok = True
    gi = [torch.from_numpy(g).to(f"cuda:{d}") for d in devices]
    for i, cb in enumerate(c):
        blk = pool[int(cb)]
        for r in range(slices):
            want = torch.stack([caches[r][l][gi[r][i]] if mla else caches[r][l][:, gi[r][i]] for l in range(4)])
            want = want.contiguous().view(torch.uint8).reshape(-1).cpu()
            per = block_bytes // slices
            if not torch.equal(blk[r * per:(r + 1) * per], want):
                ne = (blk[r * per:(r + 1) * per] != want).nonzero()
                return _fail(f"{mode}: host block {int(cb)} slice {r} differs after offload: {ne.numel()} bytes, "
                             f"first at {int(ne[0])} of {per}")
    saved = [[t.clone() for t in kv] for kv in caches]
    for kv in caches:
        for t in kv:
            t.zero_()
    g2 = np.array([1, 2, 3, 4, 5], dtype=np.int64)
    st = grp.transfer(g2, c, True, 0, 4).status
    if st != 0:
        return _fail(f"{mode}: restore status {st}")
    for di, d in enumerate(devices):
        src_rank = 0 if mla else di
        sdev = saved[src_rank][0].device
        a = torch.from_numpy(g).to(sdev)
        b = torch.from_numpy(g2).to(f"cuda:{d}")
        for l in range(4):
            want = saved[src_rank][l][a] if mla else saved[src_rank][l][:, a]
            got = caches[di][l][b] if mla else caches[di][l][:, b]
            if not torch.equal(got.cpu(), want.cpu()):
                return _fail(f"{mode}: GPU {d} layer {l} differs after restore")
    del grp
    return bool(ok)


def peer_pull_two_gpus(devices=(0, 1)) -> bool:
    """A prefix that lives only in GPU ``devices[0]``'s pages is restored into GPU ``devices[1]`` over
    NVLink through the manager (planner fragment, peer worker, pull kernel)."""
    shape = KVShape("pp", 3, 2, 64, tokens_per_block=16)
    T = 16
    mgr = KVManager(make_model_config(shape, dp_size=2),
                    CacheConfig(tokens_per_block=T, num_cpu_blocks=64, enable_p2p_gpu=True), in_process=True)
    caches = []
    for i, d in enumerate(devices):
        kv, layout = alloc_paged_cache(shape, 64, torch.device("cuda", d), "vllm",
                                       fill="normal" if i == 0 else "zeros", seed=50)
        mgr.register_gpu_tensors(kv, layout, dp_client_id=i)
        caches.append(kv)
    mgr.start()
    mgr.wait_ready(120)
    ok = True
    try:
        tok = np.arange(10 * T, dtype=np.int64)
        owner_blocks = np.array([9, 3, 60, 1, 7, 8, 33, 21, 5, 40], dtype=np.int64)
        ok = ok and mgr.publish_gpu_blocks(tok, slots_of(owner_blocks, T), dp_client_id=0) == 10
        tid, mask = mgr.kv_task_engine.get_match(tok, None, 1)
        ok = ok and int(mask.sum()) == 10 * T
        dst = np.arange(20, 30, dtype=np.int64)
        mgr.launch(tid, slots_of(dst, T))
        ok = ok and mgr.wait(tid)[tid].status.value == "success"
        for l in range(3):
            got = caches[1][l][:, torch.from_numpy(dst).to(caches[1][l].device)].cpu()
            want = caches[0][l][:, torch.from_numpy(owner_blocks).to(caches[0][l].device)].cpu()
            ok = ok and torch.equal(got, want)
        # the owner's own get does not pull from itself; withdrawn blocks are no longer offered
        ok = ok and int(mgr.kv_task_engine.get_match(tok, None, 0)[1].sum()) == 0
        ok = ok and mgr.withdraw_gpu_blocks(owner_blocks[:4], dp_client_id=0) == []
        ok = ok and int(mgr.kv_task_engine.get_match(tok, None, 1)[1].sum()) == 0
    finally:
        mgr.shutdown()
    return bool(ok)


def layerwise_two_ranks(devices=(0, 1)) -> bool:
    """Layerwise restore on two TP ranks (SGLang layout): every rank's per-layer eventfd fires once
    and every rank's pages hold its own head slice of the host blocks."""
    C = _native.C
    shape = KVShape("l2", 4, 4, 32, tokens_per_block=16)
    caches, regs = [], []
    for d in devices:
        kv, layout = alloc_paged_cache(shape, 32, torch.device("cuda", d), "sglang", tp_size=2, fill="zeros")
        caches.append(kv)
        regs.append(register_tensors(kv, layout))
    chunk = regs[0].chunk_bytes
    bb = 2 * 4 * 2 * chunk
    pool = torch.randint(0, 256, (32, bb), dtype=torch.uint8).pin_memory()
    host = dict(base=pool.data_ptr(), layer_stride=2 * chunk, kv_stride=chunk, block_stride=bb, num_blocks=32)
    opts = dict(num_layers=4, kv_dim=2, chunk_bytes=chunk, cpu_tp_stride=bb // 2, max_blocks_per_op=64,
                notify_mode="flag", layers_per_batch=0)
    grp = C.LayerwiseGroup([r.as_native() for r in regs], host, opts)
    ids = np.arange(16, dtype=np.int64)
    rev = ids[::-1].copy()
    ok = grp.restore(ids, rev, 1).status == 0
    for rank in range(2):
        for l in range(4):
            fd = grp.eventfd_of(1, rank, l)
            ok = ok and struct.unpack("Q", os.read(fd, 8))[0] == 1
        for l in range(4):
            for k in range(2):
                got = caches[rank][k * 4 + l][:16].contiguous().view(torch.uint8).reshape(16, -1).cpu()
                base = rank * (bb // 2) + l * 2 * chunk + k * chunk
                want = pool[torch.from_numpy(rev), base:base + chunk]
                ok = ok and torch.equal(got, want)
    del grp
    return bool(ok)


def nvls_fanout_all_ranks(device: torch.device, rank: int, world: int, group=None, large: bool = False):
    """Collective over the ranks of an initialised NCCL group (one process per GPU): rank 0 reads host
    blocks once and `multimem.st` replicates them into every rank's symmetric MLA cache, laid out in two
    symmetric segments; every rank compares every byte. Returns True / False, or the string
    "skipped: ..." when the fabric offers no multicast. Every rank walks the same sequence of collectives
    whatever it finds, and nothing here waits on a peer from inside a kernel. ``large``: a DeepSeek-V3-sized
    cache (61 layers, 4.6 GB per rank, three symmetric segments) instead of the 19 MB one, so that the
    multicast mappings are exercised at the size a deployment has."""
    import torch.distributed as dist
    from ..common.storage import KVCacheLayout, KVCacheLayoutType
    from ..ops.kv_copy import HostSide, decode_status, new_status
    from ..parallel.nvls import alloc_symmetric_kv_layers, fanout_restore, wait_flag
    L, N, T, D, n = (61, 1024, 64, 576, 128) if large else (4, 64, 64, 576, 24)
    per_layer = N * T * D * 2
    seg_bytes = (2 << 30) if large else 2 * per_layer
    have = torch.ones(1, device=device)
    sym = None
    try:
        sym = alloc_symmetric_kv_layers(L, per_layer, device, group, segment_bytes=seg_bytes)
    except Exception as e:  # noqa: BLE001 - no multicast, or an older torch
        have.zero_()
        why = f"{type(e).__name__}: {e}"[:120]
    dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
    if float(have.item()) < 1.0:
        return "skipped: " + (why if sym is None else "another rank has no multicast mapping")
    ok, stage = True, "carve"
    try:
        kv = [sym.layer_tensor(l, (N, T, D), torch.bfloat16) for l in range(L)]
        reg = register_tensors(kv, KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, N, T, 1, D, is_mla=True))
        chunk = reg.chunk_bytes
        g = torch.Generator().manual_seed(5)            # the same host bytes on every rank, to compare against
        NH = n if large else N                          # host blocks
        pool = torch.randint(0, 256, (NH, L, 1, chunk), dtype=torch.uint8, generator=g)
        pool = pool.pin_memory() if rank == 0 else pool  # only the reader's copy is touched by a GPU
        host = HostSide(pool.data_ptr(), chunk, chunk, L * chunk, NH)
        rng = np.random.default_rng(1)
        gpu_blocks = rng.permutation(N)[:n].astype(np.int64)
        cpu_blocks = rng.permutation(NH)[:n].astype(np.int64)
        status = new_status(device)
        scratch = torch.zeros(1, dtype=torch.int32, device=device)
        for epoch in ((1,) if large else (1, 2)):
            stage = f"clear, epoch {epoch}"
            for t in kv:
                t.zero_()
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
            stage = f"fan-out kernel, epoch {epoch}"
            if rank == 0:
                keep = fanout_restore(sym, reg, host, gpu_blocks, cpu_blocks, epoch, scratch, status)
                torch.cuda.synchronize(device)
                ok = ok and decode_status(status) == 0
                del keep
            stage = f"flag wait, epoch {epoch}"
            ok = wait_flag(sym, epoch, timeout_s=10.0) and ok
            torch.cuda.synchronize(device)
            stage = f"compare, epoch {epoch}"
            gi = torch.from_numpy(gpu_blocks).to(device)
            bad_layers = []
            for l in range(L):
                got = kv[l][gi].contiguous().view(torch.uint8).reshape(n, -1).cpu()
                if not torch.equal(got, pool[torch.from_numpy(cpu_blocks), l, 0]):
                    bad_layers.append(l)
            if bad_layers:
                global last_failure
                last_failure = f"nvls fan-out: rank {rank} layers differ: {bad_layers[:8]} ({len(bad_layers)} of {L})"
                ok = False
            untouched = torch.from_numpy(np.setdiff1d(np.arange(N), gpu_blocks)).to(device)
            ok = ok and int(kv[0][untouched].view(torch.int16).count_nonzero()) == 0
            dist.barrier(group=group)
    except Exception as e:  # noqa: BLE001
        last_failure = f"nvls fan-out, rank {rank}, at '{stage}': {type(e).__name__}: {e}"[:240]
        import sys
        print(last_failure, file=sys.stderr, flush=True)
        ok = False
    flag = torch.tensor([1.0 if ok else 0.0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    return bool(flag.item() >= 1.0)


def nvls_manager_restore_all_ranks(device: torch.device, rank: int, world: int, group=None):
    """Collective over the ranks of an initialised NCCL group: the fan-out as a MANAGER path. Every rank
    carves an MLA cache out of a symmetric pool; rank 0 owns a KVManager for the tensor-parallel group,
    registers its tensors with the pool's multicast mapping, offloads a prefix from its own cache and
    restores it into other pages with ``get_match`` / ``launch`` / ``wait``: one PCIe read, every rank's
    cache written. Every rank then waits (bounded, on the host) for its flag and compares bytes. Returns
    True / False or "skipped: ..."; every rank walks the same collectives whatever it finds."""
    import torch.distributed as dist
    from ..common.storage import KVCacheLayout, KVCacheLayoutType
    from ..parallel.nvls import alloc_symmetric_kv_layers, wait_flag
    global last_failure
    L, N, T, D, n = 4, 64, 64, 576, 6
    per_layer = N * T * D * 2
    have = torch.ones(1, device=device)
    sym, why = None, ""
    try:
        sym = alloc_symmetric_kv_layers(L, per_layer, device, group, segment_bytes=2 * per_layer)
    except Exception as e:  # noqa: BLE001 - no multicast, or an older torch
        have.zero_()
        why = f"{type(e).__name__}: {e}"[:120]
    dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
    if float(have.item()) < 1.0:
        return "skipped: " + (why if sym is None else "another rank has no multicast mapping")
    ok, mgr = True, None
    try:
        kv = [sym.layer_tensor(l, (N, T, D), torch.bfloat16) for l in range(L)]
        g = torch.Generator().manual_seed(11)
        want = torch.randn(L, n, T, D, generator=g).to(torch.bfloat16)       # the same on every rank
        src = np.array([3, 40, 11, 7, 25, 60], dtype=np.int64)
        dst = np.array([1, 2, 50, 4, 5, 33], dtype=np.int64)
        tok = np.arange(n * T, dtype=np.int64) + 1000
        if rank == 0:
            shape = KVShape("mla-fanout", L, 1, D, use_mla=True, tokens_per_block=T)
            layout = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, N, T, 1, D, is_mla=True)
            mgr = KVManager(make_model_config(shape, tp_size=world), CacheConfig(tokens_per_block=T, num_cpu_blocks=32),
                            in_process=True)
            mgr.register_gpu_tensors(kv, layout, multicast=sym)
            mgr.start()
            mgr.wait_ready(120)
            for l in range(L):
                kv[l][torch.from_numpy(src).to(device)] = want[l].to(device)
            torch.cuda.synchronize(device)
            tid = mgr.put_async(tok, slots_of(src, T))
            ok = mgr.wait(tid, timeout=60, completely=True)[tid].status.value == "success"
        dist.barrier(group=group)
        for t in kv:
            t.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        if rank == 0:
            tid, mask = mgr.get_match(tok)
            ok = ok and int(mask.sum()) == n * T
            mgr.launch(tid, slots_of(dst, T))
            ok = mgr.wait(tid, timeout=60)[tid].status.value == "success" and ok
            w = mgr.transfer_manager.engine.worker_for(WorkerKey(0, 0), TransferType.H2D)
            ok = ok and type(w).__name__ == "NvlsFanoutWorker" and w.last_epoch == 1
        ok = wait_flag(sym, 1, timeout_s=10.0) and ok
        torch.cuda.synchronize(device)
        di = torch.from_numpy(dst).to(device)
        bad = [l for l in range(L) if not torch.equal(kv[l][di].cpu(), want[l])]
        if bad:
            last_failure = f"nvls manager path: rank {rank} layers differ: {bad}"
            ok = False
        untouched = torch.from_numpy(np.setdiff1d(np.arange(N), dst)).to(device)
        ok = ok and int(kv[0][untouched].view(torch.int16).count_nonzero()) == 0
        dist.barrier(group=group)
    except Exception as e:  # noqa: BLE001
        last_failure = f"nvls manager path: {type(e).__name__}: {e}"[:200]
        ok = False
    finally:
        if mgr is not None:
            mgr.shutdown()
    flag = torch.tensor([1.0 if ok else 0.0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    torch.cuda.synchronize(device)
    dist.barrier(group=group)
    return bool(flag.item() >= 1.0)


def multi_gpu_checks(devices=(0, 1)) -> Dict[str, bool]:
    """Every two-GPU scenario above; an exception counts as a failed check and is named."""
    out: Dict[str, bool] = {}
    cases = [("tp_group_mha", lambda: tp_group_two_gpus("mha", devices))]
    cases += [(f"tp_group_{m}", (lambda m=m: tp_group_two_gpus(m, devices))) for m in SHARED_KV_MODES]
    cases += [("peer_pull_nvlink", lambda: peer_pull_two_gpus(devices)),
              ("layerwise_two_ranks", lambda: layerwise_two_ranks(devices))]
    for name, fn in cases:
        try:
            out[name] = bool(fn())
            if not out[name]:
                out[name + "_error"] = last_failure
        except Exception as e:  # noqa: BLE001
            out[name] = False
            out[name + "_error"] = f"{type(e).__name__}: {e}"[:200]
    return out


def nvls_checks_main(out_path: str) -> int:
    """Entry point of one rank of a fresh process group (``python -m flexkv_b200.utils.selfcheck --nvls OUT``
    with RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set): runs the NVSwitch checks and writes
    their results as JSON. A benchmark runs them this way, as children, so that the multicast mappings live
    in processes of their own and end with them."""
    import json
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    res: Dict[str, object] = {}
    try:
        for name, fn in ((f"nvls_fanout_{world}_ranks", lambda: nvls_fanout_all_ranks(dev, rank, world)),
                         (f"nvls_fanout_{world}_ranks_4p6GB", lambda: nvls_fanout_all_ranks(dev, rank, world, large=True)),
                         (f"nvls_manager_restore_{world}_ranks", lambda: nvls_manager_restore_all_ranks(dev, rank, world))):
            res[name] = fn()
            if res[name] is False:
                res[name + "_error"] = last_failure
    finally:
        with open(out_path, "w") as f:
            json.dump(res, f)
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        dist.destroy_process_group()
    return 0


def run_nvls_checks_in_children(timeout_s: float = 300.0) -> Dict[str, object]:
    """Called by every rank of a running job: starts one child per rank (same RANK / WORLD_SIZE / LOCAL_RANK,
    a rendezvous port of their own), waits for it on the host and returns what the child of this rank wrote.
    A child that fails or runs out of time gives ``{"nvls_checks": False, "nvls_checks_error": ...}``."""
    import json
    import subprocess
    import sys
    import tempfile
    env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC")}
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 17)
    env["MASTER_ADDR"] = os.environ.get("MASTER_ADDR", "127.0.0.1")
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    out = os.path.join(tempfile.gettempdir(), f"flexkv_b200_nvls_{os.getpid()}.json")
    try:
        proc = subprocess.run([sys.executable, "-m", "flexkv_b200.utils.selfcheck", "--nvls", out], env=env,
                              capture_output=True, text=True, timeout=timeout_s)
        if os.path.exists(out):
            with open(out) as f:
                res = json.load(f)
            if proc.returncode != 0:
                res["nvls_checks_error"] = f"child exit code {proc.returncode}: " + proc.stderr[-300:]
            return res
        return {"nvls_checks": False, "nvls_checks_error": f"child exit code {proc.returncode}: " + proc.stderr[-300:]}
    except subprocess.TimeoutExpired:
        return {"nvls_checks": False, "nvls_checks_error": f"child still running after {timeout_s:.0f} s (killed)"}
    finally:
        try:
            os.unlink(out)
        except OSError:
            pass


if __name__ == "__main__":
    import sys
    if len(sys.argv) == 3 and sys.argv[1] == "--nvls":
        sys.exit(nvls_checks_main(sys.argv[2]))
    sys.exit("usage: python -m flexkv_b200.utils.selfcheck --nvls OUT.json   (one rank of a torch.distributed job)")

