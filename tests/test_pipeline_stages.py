"""Pipeline stages served by one manager: every stage registers its own layers, an op goes to every
stage's worker and finishes when the last one reports, all stages share one host block
(reference: flexkv/transfer/transfer_engine.py:1434-1492,1562-1613, flexkv/common/config.py:554-558)."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)])
def test_two_stages_share_blocks_and_ops_join(device):
    dev = "cpu" if device == "cpu" else torch.device(device)
    full = KVShape("pp", 6, 2, 16, tokens_per_block=T)                # 6 layers, 3 per stage
    stage_shape = KVShape("pp-stage", 3, 2, 16, tokens_per_block=T)
    model = make_model_config(full, pp_size=2)
    mgr = KVManager(model, CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    stages = []
    for s in range(2):
        kv, layout = alloc_paged_cache(stage_shape, 32, dev, "vllm", fill="normal", seed=10 + s)
        mgr.register_gpu_tensors(kv, layout, pp_rank=s)
        stages.append(kv)
    mgr.start(); mgr.wait_ready(30)
    try:
        host = mgr.transfer_manager.storage.host
        assert host.block_bytes == 6 * 2 * T * 2 * 16 * 2            # one host block holds both stages' layers
        tok = np.arange(5 * T, dtype=np.int64)
        src, dst = [3, 9, 1, 30, 12], [20, 21, 22, 23, 24]
        tid = mgr.put_async(tok, slots(src))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want = [[t[:, src].clone() for t in kv] for kv in stages]
        for kv in stages:
            for t in kv:
                t[:, dst] = 0
        tid = mgr.get_async(tok, slots(dst))
        assert mgr.wait(tid)[tid].status.value == "success"
        for s, kv in enumerate(stages):
            for l in range(3):
                assert torch.equal(kv[l][:, dst], want[s][l]), (s, l)
        # the two stages landed in different halves of the host block
        blk = host.block_view(int(mgr.kv_task_engine.cache_engine.cpu_cache_engine.match(
            __import__("flexkv_b200.common.block", fromlist=["SequenceMeta"]).SequenceMeta(tok, T)).physical_blocks[0]))
        half = host.block_bytes // 2
        s0 = stages[0][0][0, src[0]].contiguous().view(torch.uint8).cpu().numpy().reshape(-1)
        s1 = stages[1][0][0, src[0]].contiguous().view(torch.uint8).cpu().numpy().reshape(-1)
        assert (blk[:s0.size] == s0).all() and (blk[half:half + s1.size] == s1).all()
        st = mgr.transfer_manager.engine.stats_by_type
        assert st["D2H"][0] == 1 and st["D2H"][2] == 5 * host.block_bytes      # one op, bytes of both stages
    finally:
        mgr.shutdown()


def test_failure_in_one_stage_fails_the_op():
    full = KVShape("pp", 4, 2, 16, tokens_per_block=T)
    stage_shape = KVShape("pp-stage", 2, 2, 16, tokens_per_block=T)
    mgr = KVManager(make_model_config(full, pp_size=2), CacheConfig(tokens_per_block=T, num_cpu_blocks=8),
                    require_gpu=True)
    for s in range(2):
        kv, layout = alloc_paged_cache(stage_shape, 16, "cpu", "vllm", fill="normal", seed=s)
        mgr.register_gpu_tensors(kv, layout, pp_rank=s)
    mgr.start(); mgr.wait_ready(30)
    try:
        from flexkv_b200.common.transfer import TransferType, WorkerKey
        w1 = mgr.transfer_manager.engine.worker_for(WorkerKey(0, 1), TransferType.D2H)
        w1.fail_next = 1                                           # host-side injection in the second stage only
        tok = np.arange(3 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots([1, 2, 3]))
        assert mgr.wait(tid, completely=True)[tid].status.value == "failed"
        tid, mask = mgr.get_match(tok)
        assert int(mask.sum()) == 0                               # nothing half-written became visible
        mgr.cancel(tid)
    finally:
        mgr.shutdown()
