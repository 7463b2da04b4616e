"""SSD -> GPU without the host pool (DISK2D): through cuFile when it initialises,
else staged through pinned memory; both paths must restore exact bytes."""
import os

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("force_staged", ["0", "1"])
def test_get_reads_ssd_tail_straight_into_gpu(tmp_path, monkeypatch, force_staged):
    monkeypatch.setenv("FLEXKV_GDS_FORCE_STAGED", force_staged)
    dev = torch.device("cuda:0")
    shape = KVShape("g", 4, 4, 64, tokens_per_block=16)      # 64 KiB blocks, 4 KiB aligned
    T, NB = 16, 96
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=33)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=32, enable_ssd=True, enable_gds=True, num_ssd_blocks=128,
                      ssd_cache_dir=str(tmp_path))
    mgr = KVManager(make_model_config(shape), cfg)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(120)
    try:
        rng = np.random.default_rng(3)
        n = 12
        tok = rng.integers(0, 1000, size=n * T, dtype=np.int64)
        src = rng.permutation(NB)[:n].astype(np.int64)
        slot = np.repeat(src, T) * T + np.tile(np.arange(T), n)
        tid = mgr.put_async(tok, slot)
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        saved = [t.clone() for t in kv]
        # keep only the first 4 blocks on the host: the other 8 must come from SSD
        mgr._clear_cpu_cache()
        tid = mgr.put_async(tok[:4 * T], slot[:4 * T])
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        for t in kv:
            t.zero_()
        tid, mask = mgr.get_match(tok)
        assert int(mask.sum()) == n * T
        graph = mgr.kv_task_engine.tasks[tid].graph
        kinds = sorted(o.transfer_type.value for o in graph.ops())
        assert kinds == ["DISK2D", "H2D", "Virtual"]
        dst = rng.permutation(NB)[:n].astype(np.int64)
        mgr.launch(tid, np.repeat(dst, T) * T + np.tile(np.arange(T), n))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        torch.cuda.synchronize()
        s, d = torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev)
        for l in range(shape.num_layers):
            assert torch.equal(kv[l][:, d], saved[l][:, s])
    finally:
        mgr.shutdown()
