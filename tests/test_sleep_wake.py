"""Suspend / resume of GPU mappings (engine sleep mode): GPU ops park while suspended, the host
tier keeps its contents, and transfers continue into re-created tensors after wake
(reference: flexkv/transfer/transfer_engine.py:1661-1716, flexkv/server/client.py:351-364,464-480)."""
import time

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_gets_park_while_suspended_and_land_in_the_new_tensors(device):
    dev = "cpu" if device == "cpu" else torch.device(device)
    shape = KVShape("z", 2, 2, 16, tokens_per_block=T)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 32, dev, "vllm", fill="normal", seed=4)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    try:
        tok = np.arange(5 * T, dtype=np.int64)
        src = [3, 9, 1, 30, 12]
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want = [t[:, src].clone() for t in kv]
        assert mgr.suspend_gpu_mappings(timeout=10)
        # the engine drops its cache (sleep); a get issued now must not touch any GPU memory
        old, old_copy = kv, [t.clone() for t in kv]
        tid = mgr.get_async(tok, slots(range(20, 25)))
        time.sleep(0.2)
        r = mgr.wait(tid, timeout=0.2)[tid]
        assert r.status.value in ("timeout", "unready", "running"), r
        # wake with freshly allocated tensors of the same geometry
        kv2, layout2 = alloc_paged_cache(shape, 32, dev, "vllm", fill="zeros")
        mgr.resume_gpu_mappings(kv2, layout2)
        assert mgr.wait(tid, timeout=10)[tid].status.value == "success"
        for l in range(2):
            assert torch.equal(kv2[l][:, 20:25], want[l])
            assert torch.equal(old[l], old_copy[l])                     # the old tensors were left alone
        # puts work against the new tensors as well
        tid = mgr.put_async(tok + 500, slots(range(5)))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
    finally:
        mgr.shutdown()
