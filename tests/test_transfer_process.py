"""The data plane in a child process: graphs go down a pipe and completions come back; a child that
is killed with work in flight makes the parent report FAILED (not a timeout) and clean up after it;
SIGTERM lets the child unpin and leave; the child leaves by itself when its parent is gone.
No GPU is involved: the ops are host <-> SSD, the failure is a killed process."""
import os
import signal
import subprocess
import sys
import time

import numpy as np

from flexkv_b200 import CacheConfig
from flexkv_b200.common.debug import install_crash_diagnostics
from flexkv_b200.common.transfer import TransferOp, TransferOpGraph, TransferType
from flexkv_b200.models import KVShape, make_model_config
from flexkv_b200.transfer_process import TransferManagerProcessHandle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _handle(tmp_path, **kw):
    shape = KVShape("p", 2, 2, 32, tokens_per_block=16)
    cfg = CacheConfig(tokens_per_block=16, num_cpu_blocks=64, enable_ssd=True, num_ssd_blocks=64,
                      ssd_cache_dir=str(tmp_path), **kw)
    h = TransferManagerProcessHandle(make_model_config(shape), cfg, require_gpu=False, sync_limit_s=2.0)
    h.start()
    t0 = time.time()
    while not h.is_ready():
        assert time.time() - t0 < 60, "child did not become ready"
        time.sleep(0.05)
    return h


def _graph(n=8):
    g = TransferOpGraph()
    ids = np.arange(n, dtype=np.int64)
    op = TransferOp(g.graph_id, TransferType.H2DISK, ids, ids)
    g.add_transfer_op(op)
    return g, op


def _collect(h, gid, limit=20.0):
    t0, recs = time.time(), []
    while time.time() - t0 < limit:
        recs += h.wait(0.2)
        if any(r.is_graph_completed() and r.graph_id == gid for r in recs):
            break
    return recs


def test_graphs_run_in_the_child_and_completions_come_back(tmp_path):
    h = _handle(tmp_path)
    try:
        assert h.alive() and h.pid != os.getpid()
        g, op = _graph()
        h.submit(g)
        recs = _collect(h, g.graph_id)
        assert [(r.op_id, r.success) for r in recs] == [(op.op_id, True), (-1, True)]
    finally:
        h.shutdown()
    assert not h.alive()


def test_killed_child_fails_its_graphs_and_its_pool_file_is_removed(tmp_path, monkeypatch):
    monkeypatch.setenv("FLEXKV_HOST_POOL_SHM", "1")       # the host pool then lives in a named file
    h = _handle(tmp_path)
    pool = h._pool_file
    assert pool and os.path.exists(pool)
    os.kill(h.pid, signal.SIGSTOP)                        # frozen: the next graph stays in flight
    g, _ = _graph()
    h.submit(g)
    os.kill(h.pid, signal.SIGKILL)
    recs = _collect(h, g.graph_id)
    done = [r for r in recs if r.is_graph_completed()]
    assert len(done) == 1 and not done[0].success and done[0].failed_graph       # FAILED, never a timeout
    assert not os.path.exists(pool)
    # later graphs fail at once instead of waiting for a process that is gone
    g2, _ = _graph()
    h.submit(g2)
    assert any(r.is_graph_completed() and not r.success for r in _collect(h, g2.graph_id, 2.0))
    h.shutdown()


def test_sigterm_lets_the_child_unpin_and_exit(tmp_path, monkeypatch):
    monkeypatch.setenv("FLEXKV_HOST_POOL_SHM", "1")
    h = _handle(tmp_path)
    pool = h._pool_file
    os.kill(h.pid, signal.SIGTERM)
    t0 = time.time()
    while h.alive() and time.time() - t0 < 20:
        time.sleep(0.05)
    assert not h.alive()
    assert not os.path.exists(pool)                       # removed by the child's own shutdown path
    h.shutdown()


def test_child_leaves_when_its_parent_dies(tmp_path):
    code = f"""
import os, sys, time
sys.path.insert(0, {ROOT!r})
from flexkv_b200 import CacheConfig
from flexkv_b200.models import KVShape, make_model_config
from flexkv_b200.transfer_process import TransferManagerProcessHandle
h = TransferManagerProcessHandle(make_model_config(KVShape("p", 2, 2, 32, tokens_per_block=16)),
                                 CacheConfig(tokens_per_block=16, num_cpu_blocks=16), require_gpu=False, sync_limit_s=1.0)
h.start()
while not h.is_ready():
    time.sleep(0.05)
print(h.pid, flush=True)
os._exit(0)          # the parent dies without a word
"""
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    child = int(out.stdout.strip().splitlines()[-1])
    t0 = time.time()
    while time.time() - t0 < 30:
        try:
            os.kill(child, 0)
        except ProcessLookupError:
            break
        time.sleep(0.1)
    else:
        os.kill(child, signal.SIGKILL)
        raise AssertionError("the transfer manager process outlived its parent")


def test_crash_diagnostics_print_thread_stacks_on_demand():
    code = ("import os, signal, sys, time\n"
            f"sys.path.insert(0, {ROOT!r})\n"
            "from flexkv_b200.common.debug import install_crash_diagnostics\n"
            "assert install_crash_diagnostics() and install_crash_diagnostics()\n"
            "os.kill(os.getpid(), signal.SIGUSR1)\n"
            "time.sleep(0.2)\n"
            "os.kill(os.getpid(), signal.SIGSEGV)\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60)
    assert out.returncode == -signal.SIGSEGV
    assert out.stderr.count("most recent call first") >= 2 and "Segmentation fault" in out.stderr
