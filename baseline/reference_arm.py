"""Reference arm of ``bench.py``: the unmodified reference KV manager (installed by
``baseline/build_reference.py`` into ``baseline/_ref``) on the headline workload.

Nothing of this repository's package, kernels or engine is imported here. The arm drives the
reference through its own public API and stock code path, as its ``benchmarks/benchmark_single_batch.py``
does: ``KVManager`` (in-process task engine, its TransferManager and worker processes), a
``KVTPClient.register_to_server`` of the paged GPU cache, then per step

    put_match x requests -> launch(as_batch=True) -> wait(completely=True)
    get_match x requests -> launch(as_batch=True) -> wait

on the same shape as the other arm: Llama-3-8B KV in the vLLM paged layout (32 layers, 8 KV heads,
head 128, bf16, 16-token blocks), 32,768 GPU blocks, 32 requests x 8,192 tokens per step, random
non-contiguous GPU block ids, N(0,1) values, one manager per GPU (weak scaling).

Timing. The reference launches its kernels in worker processes, so CUDA events of this process cannot
bracket them. ``value`` is built from the reference's own per-op transfer time (``xfer=`` of its
``[XFER]`` trace lines, ``FLEXKV_TRANSFER_TRACE=1``: launch to stream-synchronised completion, measured
by its worker); ``e2e`` is the host clock around the public API calls, exactly as for the other arm.

Two defaults of the reference are overridden for the shared GPU hosts: ``FLEXKV_ENABLE_MPS=0`` (its
default starts an MPS control daemon that would outlive the run) and a per-rank IPC endpoint.
"""
from __future__ import annotations

import json
import os
import re
import statistics
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
SHIM_PY = os.path.join(HERE, "shims", "py")

METRIC = "KV get/put GB/s per GPU & whole box at 1/2/4/8 B200; p50 get latency/8K tok"
XFER_RE = re.compile(r"\[XFER\] op=(\d+) type=(\w+) nb=(\d+) bytes=(\d+) .*? xfer=([0-9.]+)ms e2e=([0-9.]+)ms")


def unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}))


class FdCapture:
    """Send this process's stdout/stderr (and those of the children it spawns) to a file, so the
    reference's ``[XFER]`` lines, which its TransferManager process logs, can be read back."""

    def __init__(self, path: str) -> None:
        self.path = path
        self.saved = None

    def __enter__(self):
        sys.stdout.flush()
        sys.stderr.flush()
        self.saved = (os.dup(1), os.dup(2))
        fd = os.open(self.path, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o644)
        os.dup2(fd, 1)
        os.dup2(fd, 2)
        os.close(fd)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        sys.stderr.flush()
        os.dup2(self.saved[0], 1)
        os.dup2(self.saved[1], 2)
        os.close(self.saved[0])
        os.close(self.saved[1])
        return False


def run(args, ClockSampler) -> int:
    if not os.path.isfile(os.path.join(REF_DIR, "flexkv", "c_ext.so")):
        unavailable("baseline/_ref is empty: run python baseline/build_reference.py first")
        return 0

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", world))

    os.environ["PYTHONPATH"] = os.pathsep.join([REF_DIR, SHIM_PY, os.environ.get("PYTHONPATH", "")])
    os.environ["FLEXKV_ENABLE_MPS"] = "0"
    os.environ["FLEXKV_TRANSFER_TRACE"] = "1"
    os.environ.setdefault("FLEXKV_LOG_LEVEL", "INFO")
    os.environ["FLEXKV_SERVER_RECV_PORT"] = f"ipc:///tmp/flexkv_ref_{os.getpid()}_{rank}"
    sys.path[:0] = [REF_DIR, SHIM_PY]

    import numpy as np
    import torch
    import torch.distributed as dist

    try:
        from flexkv.common.config import CacheConfig, ModelConfig
        from flexkv.common.storage import KVCacheLayout, KVCacheLayoutType
        from flexkv.kvmanager import KVManager
        from flexkv.kvtask import KVResponseStatus
        from flexkv.server.client import KVTPClient
    except Exception as e:  # noqa: BLE001
        unavailable(f"reference package does not import: {type(e).__name__}: {e}")
        return 0

    if not torch.cuda.is_available():
        unavailable("no GPU visible to the reference arm")
        return 0
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("gloo")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    L, H, D, T = 32, 8, 128, 16
    blocks_per_req = args.tokens // T
    blocks_per_batch = blocks_per_req * args.requests
    block_bytes = L * 2 * T * H * D * 2
    batch_bytes = blocks_per_batch * block_bytes
    if blocks_per_batch > args.gpu_blocks:
        raise SystemExit("a batch does not fit in the GPU pool")

    avail = 0
    with open("/proc/meminfo") as f:
        for line in f:
            if line.startswith("MemAvailable"):
                avail = int(line.split()[1]) * 1024
    cap = int(avail * 0.55 / max(1, local_world))
    pool_bytes = min(int(args.host_pool_gib * 2**30), cap)
    num_cpu_blocks = int(max(pool_bytes // (block_bytes + block_bytes // 64), 2 * blocks_per_batch + 64))

    model_config = ModelConfig(num_layers=L, num_kv_heads=H, head_size=D, dtype=torch.bfloat16, tp_size=1, dp_size=1)
    cache_config = CacheConfig(tokens_per_block=T, enable_cpu=True, enable_ssd=False, num_cpu_blocks=num_cpu_blocks)
    cache_config.num_gpu_blocks = args.gpu_blocks

    log_path = os.path.join(tempfile.gettempdir(), f"flexkv_ref_arm_{os.getpid()}.log")
    open(log_path, "w").close()
    capture = FdCapture(log_path)

    def read_xfer(offset: int):
        with open(log_path, "r", errors="replace") as f:
            f.seek(offset)
            text = f.read()
            end = f.tell()
        rows = [(m.group(2), int(m.group(3)), int(m.group(4)), float(m.group(5)))
                for m in XFER_RE.finditer(text)]
        return rows, end

    t_setup = time.perf_counter()
    result = None
    err = None
    mgr = None
    with capture:
        try:
            layout = KVCacheLayout(type=KVCacheLayoutType.LAYERFIRST, num_layer=L, num_block=args.gpu_blocks,
                                   tokens_per_block=T, num_head=H, head_size=D, kv_dim=2)
            g = torch.Generator(device=dev)
            g.manual_seed(1234 + rank)
            kv = []
            for _ in range(L):
                t = torch.empty(tuple(layout.kv_shape[1:]), dtype=torch.bfloat16, device=dev)
                t.normal_(generator=g)
                kv.append(t)
            mgr = KVManager(model_config, cache_config)
            mgr.start()
            tp_client = KVTPClient(mgr.gpu_register_port, 0, local_rank, intra_client_id=0)
            tp_client.register_to_server(kv, layout)
            t_dead = time.time() + 1800
            while not mgr.is_ready():
                if time.time() > t_dead:
                    raise RuntimeError("reference manager did not become ready in 1800 s")
                time.sleep(0.5)
            setup_s = time.perf_counter() - t_setup
            vocab = 128256
            tok_bytes = block_bytes // T

            def check(res, what):
                for rsp in res.values():
                    if rsp.status != KVResponseStatus.SUCCESS:
                        raise RuntimeError(f"{what} failed: {rsp.status}")

            def one_step(seed: int):
                r = np.random.default_rng(seed)
                toks = [r.integers(0, vocab, size=args.tokens, dtype=np.int64) for _ in range(args.requests)]
                gb = r.permutation(args.gpu_blocks)[:blocks_per_batch].astype(np.int64)
                slots = [(np.repeat(gb[i * blocks_per_req:(i + 1) * blocks_per_req], T) * T +
                          np.tile(np.arange(T), blocks_per_req)) for i in range(args.requests)]
                t0 = time.perf_counter()
                ids = []
                for t in toks:
                    tid, _ = mgr.put_match(t)
                    ids.append(tid)
                bid = mgr.launch(ids, slots, as_batch=True)
                check(mgr.wait(bid, timeout=600, completely=True), "put")
                t1 = time.perf_counter()
                gb2 = r.permutation(args.gpu_blocks)[:blocks_per_batch].astype(np.int64)
                slots2 = [(np.repeat(gb2[i * blocks_per_req:(i + 1) * blocks_per_req], T) * T +
                           np.tile(np.arange(T), blocks_per_req)) for i in range(args.requests)]
                t2 = time.perf_counter()
                ids = []
                for t in toks:
                    tid, mask = mgr.get_match(t)
                    if int(np.asarray(mask).sum()) != args.tokens:
                        raise RuntimeError("get_match did not find the batch that was just put")
                    ids.append(tid)
                bid = mgr.launch(ids, slots2, as_batch=True)
                check(mgr.wait(bid, timeout=600), "get")
                t3 = time.perf_counter()
                return (t1 - t0), (t3 - t2)

            for w in range(args.warmup):
                one_step(10_000 * (rank + 1) + w)
            barrier()
            time.sleep(0.2)
            _, off = read_xfer(0)
            sampler = ClockSampler(local_rank)
            sampler.start()
            t0 = time.perf_counter()
            put_s = get_s = 0.0
            for s in range(args.steps):
                a, b = one_step(20_000 * (rank + 1) + s)
                put_s += a
                get_s += b
            barrier()
            wall_s = time.perf_counter() - t0
            clocks = sampler.stop()
            time.sleep(0.5)      # the TransferManager process logs a completed op after the waiter returns
            rows, off = read_xfer(off)
            d2h_ms = sum(x for ty, nb, by, x in rows if ty == "D2H")
            h2d_ms = sum(x for ty, nb, by, x in rows if ty == "H2D")
            d2h_bytes = sum(by for ty, nb, by, x in rows if ty == "D2H")
            h2d_bytes = sum(by for ty, nb, by, x in rows if ty == "H2D")

            # byte check of one put -> get round trip (untimed)
            r = np.random.default_rng(31337 + rank)
            n8k = 8192 // T
            tok = r.integers(0, vocab, size=8192, dtype=np.int64)
            src = r.permutation(args.gpu_blocks)[:2 * n8k].astype(np.int64)
            slot_a = np.repeat(src[:n8k], T) * T + np.tile(np.arange(T), n8k)
            slot_b = np.repeat(src[n8k:], T) * T + np.tile(np.arange(T), n8k)
            tid = mgr.put_async(tok, slot_a)
            check(mgr.wait(tid, timeout=60, completely=True), "verify put")
            tid, _ = mgr.get_match(tok)
            mgr.launch(tid, slot_b)
            check(mgr.wait(tid, timeout=60), "verify get")
            torch.cuda.synchronize()
            ia = torch.from_numpy(src[:n8k]).to(dev)
            ib = torch.from_numpy(src[n8k:]).to(dev)
            verified = all(bool(torch.equal(kv[l][:, ia], kv[l][:, ib])) for l in (0, L // 2, L - 1))

            # p50 latency of one 8K-token get through the public API
            lat = []
            r = np.random.default_rng(777 + rank)
            for i in range(args.latency_iters + 3):
                tok = r.integers(0, vocab, size=8192, dtype=np.int64)
                gb = r.permutation(args.gpu_blocks)[:n8k].astype(np.int64)
                slot = np.repeat(gb, T) * T + np.tile(np.arange(T), n8k)
                tid = mgr.put_async(tok, slot)
                check(mgr.wait(tid, timeout=60, completely=True), "latency put")
                torch.cuda.synchronize()
                t1 = time.perf_counter()
                tid, mask = mgr.get_match(tok)
                mgr.launch(tid, slot)
                rsp = mgr.wait(tid, timeout=60)[tid]
                dt = (time.perf_counter() - t1) * 1e3
                if rsp.status != KVResponseStatus.SUCCESS or int(np.asarray(rsp.return_mask).sum()) != 8192:
                    raise RuntimeError("latency probe get failed")
                if i >= 3:
                    lat.append(dt)
            p50 = statistics.median(lat)
            result = dict(put_s=put_s, get_s=get_s, wall_s=wall_s, d2h_ms=d2h_ms, h2d_ms=h2d_ms,
                          d2h_bytes=d2h_bytes, h2d_bytes=h2d_bytes, n_xfer=len(rows), p50=p50,
                          clocks=clocks, setup_s=setup_s, verified=verified, tok_bytes=tok_bytes)
        except Exception as e:  # noqa: BLE001
            import traceback
            traceback.print_exc()
            err = f"{type(e).__name__}: {e}"
        finally:
            if mgr is not None:
                try:
                    mgr.shutdown()
                except Exception:  # noqa: BLE001
                    pass

    ok = 1.0 if result is not None else 0.0
    all_ok = ok if world == 1 else -max_over_ranks(-ok)
    if all_ok < 1.0:
        if err is not None:
            sys.stderr.write(f"[reference arm rank {rank}] {err}\n")
            try:
                with open(log_path, "r", errors="replace") as f:
                    sys.stderr.write(f.read()[-6000:])
            except OSError:
                pass
        if rank == 0:
            unavailable(f"reference arm failed at run time: {err or 'another rank failed'}"[:300])
        if world > 1:
            dist.destroy_process_group()
        return 0

    steps = args.steps
    want = batch_bytes * steps
    xfer_ok = result["d2h_bytes"] == want and result["h2d_bytes"] == want and result["d2h_ms"] > 0 and result["h2d_ms"] > 0
    d2h_ms = max_over_ranks(result["d2h_ms"] if xfer_ok else float("inf"))
    h2d_ms = max_over_ranks(result["h2d_ms"] if xfer_ok else float("inf"))
    put_s, get_s = max_over_ranks(result["put_s"]), max_over_ranks(result["get_s"])
    wall_s = max_over_ranks(result["wall_s"])
    p50 = max_over_ranks(result["p50"])
    verified = -max_over_ranks(-(1.0 if result["verified"] else 0.0)) >= 1.0
    if rank == 0:
        e2e_val = 2 * want * world / (put_s + get_s) / 1e9
        if d2h_ms != float("inf"):
            kernel_ms = d2h_ms + h2d_ms
            value = 2 * want * world / (kernel_ms * 1e-3) / 1e9
            unit = "GB/s (put+get bytes / the reference workers' own transfer time, all GPUs)"
            put_gbs, get_gbs = want / (d2h_ms * 1e-3) / 1e9, want / (h2d_ms * 1e-3) / 1e9
        else:
            kernel_ms = (put_s + get_s) * 1e3
            value = e2e_val
            unit = "GB/s (put+get bytes / host time through the public API; no [XFER] lines were read)"
            put_gbs, get_gbs = want / put_s / 1e9, want / get_s / 1e9
        out = {
            "metric": METRIC, "impl": "reference", "value": round(value, 2), "unit": unit,
            "n_gpus": world, "steps": steps, "warmup": args.warmup, "ms_per_step": round(kernel_ms / steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform token ids, N(0,1) KV, random-init",
            "put_gbs_per_gpu": round(put_gbs, 2), "get_gbs_per_gpu": round(get_gbs, 2),
            "region_ms_per_step": round(wall_s * 1e3 / steps, 3),
            "p50_get_latency_ms_8k_tokens": round(p50, 3),
            "e2e": {"value": round(e2e_val, 2), "unit": "GB/s", "ms_per_step": round((put_s + get_s) * 1e3 / steps, 2),
                    "h2d_bytes_per_step": batch_bytes + 2 * blocks_per_batch * 8, "d2h_bytes_per_step": batch_bytes + 8,
                    "api": "flexkv.KVManager.put_match/get_match/launch(as_batch)/wait"},
            "gpu_launches": 2 * steps * world, "clocks": result["clocks"],
            "verified": {"put_get_roundtrip_bytes": verified},
            "config": {"model": "llama3-8b KV, vLLM paged layout", "global_batch": args.requests * world,
                       "seq_len": args.tokens, "parallelism": f"dp{world}", "gpu_blocks": args.gpu_blocks,
                       "host_pool_gib": round(num_cpu_blocks * block_bytes / 2**30, 1),
                       "host_pool_gib_requested": args.host_pool_gib, "block_bytes": block_bytes,
                       "bytes_per_step_per_gpu": 2 * batch_bytes,
                       "l2": "inputs larger than L2 (32 GiB per direction per step)",
                       "host_codec": "none", "engine": "reference transfer.cu, 4 CTAs x 1024 threads (its defaults)",
                       "build": "baseline/_ref from baseline/build_reference.py", "setup_s": round(result["setup_s"], 1)},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    try:
        os.unlink(log_path)
    except OSError:
        pass
    return 0
