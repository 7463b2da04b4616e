"""Request tracer and replay (reference: flexkv/common/tracer.py:13-333, tests/replay_from_tracer.py)."""
import json

import numpy as np

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.common.config import GLOBAL_CONFIG_FROM_ENV
from flexkv_b200.common.trace_replay import read_trace, replay
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

T = 4


def slots(blocks):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def test_trace_is_written_and_replays_with_the_same_hits(tmp_path, monkeypatch):
    path = str(tmp_path / "trace.log")
    env = GLOBAL_CONFIG_FROM_ENV
    monkeypatch.setattr(env, "enable_trace", True)
    monkeypatch.setattr(env, "trace_file_path", path)
    shape = KVShape("tr", 2, 2, 16, tokens_per_block=T)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=16), require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 32, "cpu", "vllm", fill="normal", seed=1)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start(); mgr.wait_ready(30)
    tok = np.arange(6 * T, dtype=np.int64)
    tid = mgr.put_async(tok, slots(range(6)))
    mgr.wait(tid, completely=True)
    tid, mask = mgr.get_match(np.concatenate([tok[:4 * T], np.arange(100, 100 + 2 * T)]))
    hit = int(mask.sum())
    assert hit == 4 * T
    mgr.launch(tid, slots(range(10, 14)))
    mgr.wait(tid)
    tid2, mask2 = mgr.get_match(np.arange(500, 500 + 3 * T))
    assert int(mask2.sum()) == 0
    mgr.shutdown()
    monkeypatch.setattr(env, "enable_trace", False)

    recs = list(read_trace(path))
    kinds = [r["type"] for r in recs]
    assert kinds[0] == "CONFIG" and "PUT" in kinds and kinds.count("GET_MATCH") == 2 and "LAUNCH" in kinds
    assert "password" not in json.dumps(recs[0])
    st = replay(recs)
    assert st["put"] == 1 and st["get_match"] == 2 and st["launch"] == 1 and st["failed"] == 0
    assert st["get_hit_tokens"] == hit and st["get_query_tokens"] == 6 * T + 3 * T
    # a smaller host pool changes the outcome of the same trace
    st2 = replay(recs, cache_overrides={"num_cpu_blocks": 2})
    assert st2["get_hit_tokens"] < hit
