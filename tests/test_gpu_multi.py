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
from flexkv_b200.utils import selfcheck

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
    assert selfcheck.tp_group_two_gpus(mode)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_peer_pull_across_gpus_through_kvmanager():
    assert selfcheck.peer_pull_two_gpus()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_layerwise_two_ranks_each_signals_its_own_layers():
    assert selfcheck.layerwise_two_ranks()


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
