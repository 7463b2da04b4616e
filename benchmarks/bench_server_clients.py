#!/usr/bin/env python
"""Request rate of ONE KVServer (one index, one planner, one scheduler) under several data-parallel clients,
on the CPU: every client is a thread with a KVDPClient of its own that puts and then gets 8K-token requests;
the data plane's workers complete at once, so the figure is the server's control plane (ZeroMQ hop, hash,
match, plan, graph scheduling, completion, reply) and how it shares one interpreter between the clients.
The same requests through private in-process managers are the comparison.
(Reference counterpart: its dp_size > 1 mode, flexkv/kvmanager.py:69-107, flexkv/server/server.py.)"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import CacheConfig, KVManager, KVTPClient  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config  # noqa: E402
from flexkv_b200.server.utils import unique_ipc_endpoint  # noqa: E402
from flexkv_b200.transfer import workers as W  # noqa: E402

T = 16


def client_loop(mgr, toks, out):
    slot = np.arange(8192, dtype=np.int64)
    lat_put, lat_get = [], []
    for tok in toks:
        t0 = time.perf_counter()
        tid = mgr.put_async(tok, slot)
        mgr.wait(tid, completely=True)
        lat_put.append(time.perf_counter() - t0)
    for tok in toks:
        t0 = time.perf_counter()
        tid, mask = mgr.get_match(tok)
        mgr.launch(tid, slot[mask])
        mgr.wait(tid)
        lat_get.append(time.perf_counter() - t0)
    out.append((lat_put, lat_get))


def run(n_clients, requests, shared):
    shape = KVShape("tiny", 1, 1, 8, tokens_per_block=T)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=max(1 << 17, n_clients * requests * 512))
    mgrs = []
    if shared:
        model = make_model_config(shape, dp_size=n_clients)
        ep, reg = unique_ipc_endpoint("bsrv"), unique_ipc_endpoint("breg")
        for d in range(n_clients):
            mgrs.append(KVManager(model, cache, dp_client_id=d, server_recv_port=ep, gpu_register_port=reg,
                                  require_gpu=(d == 0) or None))
        keep = []
        for d in range(n_clients):
            kv, layout = alloc_paged_cache(shape, 1024, "cpu", "vllm", fill="zeros")
            KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout, mode="same_process")
            keep.append(kv)
    else:
        keep = []
        for d in range(n_clients):
            m = KVManager(make_model_config(shape), cache, require_gpu=True)
            kv, layout = alloc_paged_cache(shape, 1024, "cpu", "vllm", fill="zeros")
            m.register_gpu_tensors(kv, layout)
            keep.append(kv)
            mgrs.append(m)
    for m in mgrs:
        m.start()
    for m in mgrs:
        m.wait_ready(60)
    rng = np.random.default_rng(7)
    work = [[rng.integers(0, 128256, size=8192, dtype=np.int64) for _ in range(requests)] for _ in range(n_clients)]
    out, threads = [], []
    t0 = time.perf_counter()
    for m, toks in zip(mgrs, work):
        th = threading.Thread(target=client_loop, args=(m, toks, out))
        th.start()
        threads.append(th)
    for th in threads:
        th.join()
    wall = time.perf_counter() - t0
    for m in reversed(mgrs):
        m.shutdown()
    puts = [x for lp, _ in out for x in lp]
    gets = [x for _, lg in out for x in lg]
    p = lambda v, q: round(sorted(v)[int(q * (len(v) - 1))] * 1e3, 3)   # noqa: E731
    return dict(mode="one server" if shared else "private managers", clients=n_clients, requests_per_client=requests,
                requests_per_s=round(2 * n_clients * requests / wall, 1), put_ms_p50=p(puts, 0.5), put_ms_p99=p(puts, 0.99),
                get_ms_p50=p(gets, 0.5), get_ms_p99=p(gets, 0.99))


def child_main(a):
    """One data-parallel client in a process of its own, against a server that runs elsewhere."""
    from flexkv_b200.common.config import GLOBAL_CONFIG_FROM_ENV
    GLOBAL_CONFIG_FROM_ENV.server_launch_mode = "external"
    GLOBAL_CONFIG_FROM_ENV.server_client_mode = True          # also with one client: the point is the server hop
    shape = KVShape("tiny", 1, 1, 8, tokens_per_block=T)
    model = make_model_config(shape, dp_size=a.dp_size)
    cache = CacheConfig(tokens_per_block=T, num_cpu_blocks=a.cpu_blocks)
    mgr = KVManager(model, cache, dp_client_id=a.child, server_recv_port=a.ep, gpu_register_port=a.reg)
    mgr.start()
    mgr.wait_ready(120)
    rng = np.random.default_rng(100 + a.child)
    toks = [rng.integers(0, 128256, size=8192, dtype=np.int64) for _ in range(a.requests)]
    # every client starts its timed part at the same wall-clock second
    time.sleep(max(0.0, a.start_at - time.time()))
    out = []
    t0 = time.perf_counter()
    client_loop(mgr, toks, out)
    wall = time.perf_counter() - t0
    print("CHILD " + json.dumps(dict(wall=wall, put=out[0][0], get=out[0][1])), flush=True)
    mgr.shutdown()


def run_processes(n_clients, requests):
    """The server in one process, every client in another: what a deployment with one engine process per DP
    rank looks like. The server's workers run the CPU stand-in of the copy kernel (1,024 scattered 256-byte
    copies per request), so the figure includes a data plane that is not free."""
    import subprocess
    import tempfile
    from flexkv_b200.common.memory_handle import alloc_shared_host_tensor
    shape = KVShape("tiny", 1, 1, 8, tokens_per_block=T)
    blocks = max(1 << 17, n_clients * requests * 512)
    ep, reg = unique_ipc_endpoint("psrv"), unique_ipc_endpoint("preg")
    mcfg = dict(num_layers=1, num_kv_heads=1, head_size=8, dtype="bfloat16", dp_size=n_clients)
    ccfg = dict(tokens_per_block=T, num_cpu_blocks=blocks)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    srv = subprocess.Popen([sys.executable, "-m", "flexkv_b200.server", "--model-config", json.dumps(mcfg),
                            "--cache-config", json.dumps(ccfg), "--recv-endpoint", ep, "--gpu-register-port", reg,
                            "--no-gpu"], cwd=root, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    tmp = tempfile.mkdtemp(prefix="flexkv_bsc_", dir="/dev/shm")
    kids = []
    try:
        t0 = time.time()
        while not os.path.exists(reg[len("ipc://"):]) and time.time() - t0 < 60:
            time.sleep(0.05)
        keep = []
        for d in range(n_clients):
            src, layout = alloc_paged_cache(shape, 1024, "cpu", "vllm", fill="zeros")
            kv = [alloc_shared_host_tensor(t.shape, t.dtype, os.path.join(tmp, f"kv_{d}_{i}.bin")) for i, t in enumerate(src)]
            KVTPClient(reg, dp_client_id=d, device_id=0, tp_rank=0).register_to_server(kv, layout)
            keep.append(kv)
        start_at = time.time() + 6.0 + 0.5 * n_clients
        for d in range(n_clients):
            kids.append(subprocess.Popen([sys.executable, os.path.abspath(__file__), "--child", str(d), "--dp-size",
                                          str(n_clients), "--ep", ep, "--reg", reg, "--requests", str(requests),
                                          "--cpu-blocks", str(blocks), "--start-at", repr(start_at)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True))
        recs = []
        for k in kids:
            text, _ = k.communicate(timeout=600)
            line = next((l for l in text.splitlines() if l.startswith("CHILD ")), None)
            if line is None:
                raise RuntimeError("a client process gave no result")
            recs.append(json.loads(line[6:]))
    finally:
        for k in kids:
            if k.poll() is None:
                k.kill()
        srv.terminate()
        try:
            srv.wait(timeout=20)
        except subprocess.TimeoutExpired:
            srv.kill()
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
    wall = max(r["wall"] for r in recs)
    puts = [x for r in recs for x in r["put"]]
    gets = [x for r in recs for x in r["get"]]
    p = lambda v, q: round(sorted(v)[int(q * (len(v) - 1))] * 1e3, 3)   # noqa: E731
    return dict(mode="one server process, one process per client", clients=n_clients, requests_per_client=requests,
                requests_per_s=round(2 * n_clients * requests / wall, 1), put_ms_p50=p(puts, 0.5), put_ms_p99=p(puts, 0.99),
                get_ms_p50=p(gets, 0.5), get_ms_p99=p(gets, 0.99))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--clients", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--requests", type=int, default=100)
    ap.add_argument("--processes", action="store_true", help="server and clients in processes of their own")
    ap.add_argument("--child", type=int, default=-1)
    ap.add_argument("--dp-size", type=int, default=1)
    ap.add_argument("--ep", default="")
    ap.add_argument("--reg", default="")
    ap.add_argument("--cpu-blocks", type=int, default=1 << 17)
    ap.add_argument("--start-at", type=float, default=0.0)
    a = ap.parse_args()
    if a.child >= 0:
        child_main(a)
        return
    if a.processes:
        for n in a.clients:
            print(json.dumps(run_processes(n, a.requests)), flush=True)
        return
    W.HostEmulatedGpuWorker.execute = lambda self, op: W.OpOutcome(True, num_bytes=0)
    for n in a.clients:
        for shared in (False, True):
            if shared and n == 1:
                continue
            print(json.dumps(run(n, a.requests, shared)), flush=True)


if __name__ == "__main__":
    main()
