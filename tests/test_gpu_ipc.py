"""An engine worker in another process shares its GPU KV cache through CUDA IPC handles; the
manager in this process offloads and restores through the imported mappings
(reference: flexkv/server/client.py:366-496, flexkv/common/memory_handle.py:466-545)."""
import json
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, make_model_config
from flexkv_b200.server.utils import unique_ipc_endpoint

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
T = 16


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


@pytest.mark.parametrize("alloc", ["cuda_ipc", "vmm"])
def test_manager_moves_blocks_of_a_cache_owned_by_another_process(tmp_path, alloc):
    reg = unique_ipc_endpoint("ipcreg")
    shape = KVShape("ipc", 4, 4, 64, tokens_per_block=T)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=32),
                    gpu_register_port=reg, require_gpu=True)
    mgr.start()
    child = subprocess.Popen([sys.executable, os.path.join(HERE, "mp_workers", "ipc_engine_worker.py"), reg,
                              str(tmp_path), alloc], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        mgr.wait_ready(120)
        tok = np.arange(5 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots([3, 9, 1, 30, 12]))
        assert mgr.wait(tid, completely=True, timeout=60)[tid].status.value == "success"
        tid = mgr.get_async(tok, slots([40, 41, 42, 43, 44]))
        assert mgr.wait(tid, timeout=60)[tid].status.value == "success"
        open(tmp_path / "moved", "w").close()
        t0 = time.time()
        while not (tmp_path / "result.json").exists() and time.time() - t0 < 60:
            time.sleep(0.05)
        res = json.loads((tmp_path / "result.json").read_text())
        assert res == {"ok": True, "untouched": True}
    finally:
        mgr.shutdown()                                  # the importer lets go before the owner frees
        open(tmp_path / "exit", "w").close()
        try:
            out, _ = child.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            child.kill()
            out, _ = child.communicate()
    assert child.returncode == 0, out[-2000:]
