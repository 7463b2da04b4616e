"""Replays a request trace written by ``FlexKVTracer`` against a fresh KVManager.

``python -m flexkv_b200.common.trace_replay trace.log [--gpu-blocks N] [--device cpu|cuda:0]``

The CONFIG record rebuilds the model and cache configuration (tier sizes may be overridden),
a paged cache of the traced geometry is allocated as the engine's stand-in, and every
PUT / GET / PUT_MATCH / GET_MATCH / PREFETCH / LAUNCH / WAIT / RESET record is issued in order
with the traced task ids mapped onto the new ones. Reports per-kind counts, hit tokens and wall
time, so that an eviction policy, a pool size or a code change can be judged on a production
trace (reference tool: tests/replay_from_tracer.py).
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Any, Dict, Iterable, Optional

import numpy as np
import torch

_DTYPES = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16, "torch.float32": torch.float32,
           "torch.uint8": torch.uint8, "torch.float8_e4m3fn": torch.float8_e4m3fn}


def read_trace(path: str) -> Iterable[Dict[str, Any]]:
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                yield json.loads(line)


def _np(a, dtype=np.int64) -> Optional[np.ndarray]:
    return None if a is None else np.asarray(a, dtype=dtype)


def replay(records: Iterable[Dict[str, Any]], device: str = "cpu", gpu_blocks: int = 0,
           cache_overrides: Optional[Dict[str, Any]] = None, wait_timeout: float = 60.0) -> Dict[str, Any]:
    from .. import CacheConfig, KVManager
    from ..common.config import ModelConfig
    from ..models import KVShape, alloc_paged_cache
    mgr = None
    idmap: Dict[int, int] = {}
    stats = dict(records=0, put=0, get=0, put_match=0, get_match=0, prefetch=0, launch=0, wait=0, reset=0,
                 get_hit_tokens=0, get_query_tokens=0, put_new_tokens=0, failed=0)
    max_slot = [0]
    recs = list(records)
    for r in recs:                                   # the stand-in cache must cover every traced slot
        for key in ("slot_mapping",):
            if r.get(key):
                max_slot[0] = max(max_slot[0], max(r[key]))
        for sm in r.get("slot_mappings") or []:
            if sm:
                max_slot[0] = max(max_slot[0], max(sm))
    t0 = time.perf_counter()
    try:
        for r in recs:
            stats["records"] += 1
            kind = r.get("type")
            if kind == "CONFIG":
                if mgr is not None:
                    continue
                mc_d, cc_d = dict(r["model_config"]), dict(r.get("cache_config") or {})
                mc_d["dtype"] = _DTYPES.get(str(mc_d.get("dtype")), torch.bfloat16)
                mc_fields = {f for f in ModelConfig.__dataclass_fields__}
                mc = ModelConfig(**{k: v for k, v in mc_d.items() if k in mc_fields and v is not None
                                    and not isinstance(v, str) or k == "dtype"})
                cc_fields = {f for f in CacheConfig.__dataclass_fields__}
                cc_kw = {k: v for k, v in cc_d.items() if k in cc_fields and k != "swa"
                         and not (isinstance(v, str) and v.startswith("<"))}
                cc_kw.update(cache_overrides or {})
                cc = CacheConfig(**cc_kw)
                T = cc.tokens_per_block
                shape = KVShape("replay", mc.num_layers, mc.num_kv_heads, mc.head_size, dtype=mc.dtype,
                                use_mla=mc.use_mla, tokens_per_block=T)
                nb = max(gpu_blocks, max_slot[0] // T + 1)
                mgr = KVManager(mc, cc, require_gpu=True, in_process=True)
                kv, layout = alloc_paged_cache(shape, nb, torch.device(device) if device != "cpu" else "cpu", "vllm",
                                               fill="zeros")
                mgr.register_gpu_tensors(kv, layout)
                mgr.start()
                mgr.wait_ready(300)
                stats["gpu_blocks"] = nb
                continue
            if mgr is None:
                raise ValueError("the trace has no CONFIG record before its first request")
            ns = r.get("namespace")
            if kind == "PUT":
                stats["put"] += 1
                idmap[r["task_id"]] = mgr.put_async(_np(r["token_ids"]), _np(r["slot_mapping"]),
                                                    _np(r.get("token_mask"), np.bool_), namespace=ns)
            elif kind == "GET":
                stats["get"] += 1
                idmap[r["task_id"]] = mgr.get_async(_np(r["token_ids"]), _np(r["slot_mapping"]),
                                                    _np(r.get("token_mask"), np.bool_), namespace=ns)
            elif kind == "PUT_MATCH":
                stats["put_match"] += 1
                tid, mask = mgr.put_match(_np(r["token_ids"]), _np(r.get("token_mask"), np.bool_), namespace=ns)
                idmap[r["task_id"]] = tid
                stats["put_new_tokens"] += int(mask.sum())
            elif kind == "GET_MATCH":
                stats["get_match"] += 1
                tid, mask = mgr.get_match(_np(r["token_ids"]), _np(r.get("token_mask"), np.bool_), namespace=ns)
                idmap[r["task_id"]] = tid
                stats["get_hit_tokens"] += int(mask.sum())
                stats["get_query_tokens"] += len(r["token_ids"])
            elif kind == "PREFETCH":
                stats["prefetch"] += 1
                idmap[r["task_id"]] = mgr.prefetch_async(_np(r["token_ids"]), namespace=ns)
            elif kind == "LAUNCH":
                stats["launch"] += 1
                tids = [idmap[t] for t in r["task_ids"] if t in idmap]
                # the replayed match may differ from the traced one (other pool sizes): fit the mapping
                sms = []
                for t, sm in zip(tids, r["slot_mappings"]):
                    task = mgr.kv_task_engine.tasks.get(t)
                    need = int(np.asarray(task.return_mask).sum()) if task is not None else 0
                    sm = np.asarray(sm or [], dtype=np.int64)
                    if len(sm) < need:
                        extra = np.arange(need - len(sm), dtype=np.int64)
                        sm = np.concatenate([sm, extra])
                    sms.append(sm[:need])
                out = mgr.launch(tids, sms, as_batch=bool(r.get("as_batch")),
                                 layerwise_transfer=bool(r.get("layerwise_transfer")),
                                 counter_id=int(r.get("counter_id") or 0))
                if r.get("as_batch") and len(out) == 1:
                    for t in r["task_ids"]:
                        idmap.setdefault(("batch", t), out[0])
            elif kind == "WAIT":
                stats["wait"] += 1
                tids = [idmap[t] for t in r["task_ids"] if t in idmap]
                if tids:
                    res = mgr.wait(tids, timeout=wait_timeout, completely=bool(r.get("completely")))
                    stats["failed"] += sum(1 for v in res.values() if v.status.value not in ("success", "notfound"))
            elif kind == "RESET":
                stats["reset"] += 1
                mgr.kv_task_engine.reset_cache() if hasattr(mgr.kv_task_engine, "reset_cache") else None
    finally:
        stats["wall_s"] = round(time.perf_counter() - t0, 3)
        if mgr is not None:
            mgr.shutdown()
    if stats["get_query_tokens"]:
        stats["get_token_hit_rate"] = round(stats["get_hit_tokens"] / stats["get_query_tokens"], 4)
    return stats


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("trace")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--gpu-blocks", type=int, default=0)
    ap.add_argument("--num-cpu-blocks", type=int, default=0)
    ap.add_argument("--eviction-policy", default="")
    a = ap.parse_args()
    over: Dict[str, Any] = {}
    if a.num_cpu_blocks:
        over["num_cpu_blocks"] = a.num_cpu_blocks
    if a.eviction_policy:
        over["eviction_policy"] = a.eviction_policy
    print(json.dumps(replay(read_trace(a.trace), a.device, a.gpu_blocks, over)))


if __name__ == "__main__":
    main()
