"""Multi-GPU data plane: TP transfer group (MHA slices and shared-KV modes),
NVLink peer pull (kernel level and through KVManager), layerwise on two ranks,
NVSwitch fan-out restore (child processes under torchrun)."""
import glob
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager, _native
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
from flexkv_b200.storage.gpu_layout import register_tensors

C = _native.C
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _slots(blocks, T):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


@pytest.mark.gpu
def test_peer_copy_converts_layouts_on_one_gpu():
    """Source and destination are addressed independently: vLLM -> SGLang on the same device."""
    dev = torch.device("cuda:0")
    shape = KVShape("p", 3, 2, 64, tokens_per_block=16)
    src, lsrc = alloc_paged_cache(shape, 40, dev, "vllm", fill="normal", seed=31)
    dst, ldst = alloc_paged_cache(shape, 50, dev, "sglang", fill="zeros")
    rs, rd = register_tensors(src, lsrc), register_tensors(dst, ldst)
    cp = C.PeerCopier([rs.as_native(), rd.as_native()], 3, 2, rs.chunk_bytes, num_ctas=6, tile_bytes=2048,
                      max_blocks_per_op=64)
    sb = np.array([5, 1, 39, 7], dtype=np.int64)
    db = np.array([0, 49, 3, 20], dtype=np.int64)
    r = cp.pull(1, 0, db, sb, 0, 3)
    assert r.status == 0
    for l in range(3):
        for k in range(2):
            assert torch.equal(dst[k * 3 + l][torch.from_numpy(db).cuda()], src[l][k][torch.from_numpy(sb).cuda()])
    assert cp.pull(1, 0, np.array([99], dtype=np.int64), np.array([0], dtype=np.int64), 0, 3).status == 1


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("mode", ["mha", "sharded", "all_write", "rank0_only", "layer_parallel", "rank_rotate"])
def test_tp_group_two_gpus(mode):
    mla = mode != "mha"
    shape = KVShape("t", 4, 1 if mla else 4, 128 if mla else 32, use_mla=mla, tokens_per_block=16)
    caches, regs = [], []
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 48, torch.device("cuda", d), "vllm", tp_size=1 if mla else 2,
                                       fill="normal", seed=40 if mla else 40 + d)
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
    assert grp.transfer(g, c, False, 0, 4).status == 0
    gi = [torch.from_numpy(g).to(f"cuda:{d}") for d in range(2)]
    for i, cb in enumerate(c):
        blk = pool[int(cb)]
        for r in range(slices):
            want = torch.stack([caches[r][l][gi[r][i]] if mla else caches[r][l][:, gi[r][i]] for l in range(4)])
            want = want.contiguous().view(torch.uint8).reshape(-1).cpu()
            per = block_bytes // slices
            assert torch.equal(blk[r * per:(r + 1) * per], want), (mode, i, r)
    saved = [[t.clone() for t in kv] for kv in caches]
    for kv in caches:
        for t in kv:
            t.zero_()
    g2 = np.array([1, 2, 3, 4, 5], dtype=np.int64)
    assert grp.transfer(g2, c, True, 0, 4).status == 0
    for d in range(2):
        src_rank = 0 if mla else d
        a = torch.from_numpy(g).to(f"cuda:{d}")
        b = torch.from_numpy(g2).to(f"cuda:{d}")
        for l in range(4):
            want = (saved[src_rank][l][a.to(saved[src_rank][l].device)] if mla
                    else saved[src_rank][l][:, a.to(saved[src_rank][l].device)])
            got = caches[d][l][b] if mla else caches[d][l][:, b]
            assert torch.equal(got.cpu(), want.cpu()), (mode, d, l)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_peer_pull_across_gpus_through_kvmanager():
    shape = KVShape("pp", 3, 2, 64, tokens_per_block=16)
    T = 16
    mgr = KVManager(make_model_config(shape, dp_size=2), CacheConfig(tokens_per_block=T, num_cpu_blocks=64,
                                                                      enable_p2p_gpu=True), in_process=True)
    caches = []
    for d in range(2):
        kv, layout = alloc_paged_cache(shape, 64, torch.device("cuda", d), "vllm",
                                       fill="normal" if d == 0 else "zeros", seed=50)
        mgr.register_gpu_tensors(kv, layout, dp_client_id=d)
        caches.append(kv)
    mgr.start()
    mgr.wait_ready(120)
    try:
        tok = np.arange(10 * T, dtype=np.int64)
        owner_blocks = np.array([9, 3, 60, 1, 7, 8, 33, 21, 5, 40], dtype=np.int64)
        assert mgr.publish_gpu_blocks(tok, _slots(owner_blocks, T), dp_client_id=0) == 10
        # rank 1 asks for the prefix: nothing on host, everything in rank 0's HBM
        tid, mask = mgr.kv_task_engine.get_match(tok, None, 1)
        assert int(mask.sum()) == 10 * T
        dst = np.arange(20, 30, dtype=np.int64)
        mgr.launch(tid, _slots(dst, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        for l in range(3):
            got = caches[1][l][:, torch.from_numpy(dst).to("cuda:1")].cpu()
            want = caches[0][l][:, torch.from_numpy(owner_blocks).to("cuda:0")].cpu()
            assert torch.equal(got, want)
        # the owner's own get does not pull from itself; withdrawn blocks are no longer offered
        assert int(mgr.kv_task_engine.get_match(tok, None, 0)[1].sum()) == 0
        assert mgr.withdraw_gpu_blocks(owner_blocks[:4], dp_client_id=0) == []
        assert int(mgr.kv_task_engine.get_match(tok, None, 1)[1].sum()) == 0   # the prefix lost its head
    finally:
        mgr.shutdown()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_layerwise_two_ranks_each_signals_its_own_layers():
    import struct
    shape = KVShape("l2", 4, 4, 32, tokens_per_block=16)
    caches, regs = [], []
    for d in range(2):
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
    r = grp.restore(ids, ids[::-1].copy(), 1)
    assert r.status == 0
    for rank in range(2):
        for l in range(4):
            fd = grp.eventfd_of(1, rank, l)
            assert struct.unpack("Q", os.read(fd, 8))[0] == 1
        for l in range(4):
            for k in range(2):
                got = caches[rank][k * 4 + l][:16].contiguous().view(torch.uint8).reshape(16, -1).cpu()
                base = rank * (bb // 2) + l * 2 * chunk + k * chunk
                want = pool[torch.from_numpy(ids[::-1].copy()), base:base + chunk]
                assert torch.equal(got, want)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nvls_fanout_restore_in_child_processes(tmp_path):
    env = dict(os.environ, FKV_RESULT_DIR=str(tmp_path), PYTHONPATH=ROOT)
    n = min(torch.cuda.device_count(), 4)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29611",
           os.path.join(ROOT, "tests", "mp_workers", "nvls_fanout_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    results = [json.load(open(f)) for f in sorted(glob.glob(str(tmp_path / "nvls_rank*.json")))]
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:] + str(results)
    assert len(results) == n and all(r["ok"] for r in results), results
    if any("skipped" in r for r in results):
        pytest.skip(results[0].get("skipped", "no multicast"))
