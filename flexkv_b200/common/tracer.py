"""Request tracer: a JSON-lines file holding the configuration and every
GET / PUT / MATCH / LAUNCH / WAIT request, with size-based rotation, so that a
production trace can be replayed against a fresh KVManager
(enabled by ``FLEXKV_ENABLE_TRACE=1``; reference: flexkv/common/tracer.py:13-333,
replay tool tests/replay_from_tracer.py)."""
from __future__ import annotations

import json
import os
import threading
import time
from typing import List, Optional

import numpy as np

from .config import GLOBAL_CONFIG_FROM_ENV


def _arr(a) -> Optional[List[int]]:
    if a is None:
        return None
    return np.asarray(a).astype(np.int64).tolist()


class FlexKVTracer:
    def __init__(self, enabled: bool, path: str = "./flexkv_trace.log", max_file_size_mb: int = 100,
                 max_files: int = 5, flush_interval_ms: int = 1000) -> None:
        self.enabled = enabled
        self.path = path
        self.max_bytes = max_file_size_mb * (1 << 20)
        self.max_files = max_files
        self.flush_interval = flush_interval_ms / 1e3
        self._lock = threading.Lock()
        self._f = None
        self._last_flush = 0.0
        if enabled:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            self._f = open(path, "a", buffering=1 << 16)

    @classmethod
    def from_env(cls, model_config=None, cache_config=None) -> "FlexKVTracer":
        env = GLOBAL_CONFIG_FROM_ENV
        t = cls(env.enable_trace, env.trace_file_path, env.trace_max_file_size_mb, env.trace_max_files,
                env.trace_flush_interval_ms)
        if t.enabled and model_config is not None:
            t.trace_config(model_config, cache_config)
        return t

    def _rotate(self) -> None:
        self._f.close()
        for i in range(self.max_files - 1, 0, -1):
            src = self.path if i == 1 else f"{self.path}.{i - 1}"
            if os.path.exists(src):
                os.replace(src, f"{self.path}.{i}")
        self._f = open(self.path, "a", buffering=1 << 16)

    def _write(self, rec: dict) -> None:
        if not self.enabled:
            return
        rec["ts"] = time.time()
        line = json.dumps(rec, separators=(",", ":")) + "\n"
        with self._lock:
            if self._f is None:
                return
            self._f.write(line)
            now = time.monotonic()
            if now - self._last_flush > self.flush_interval:
                self._f.flush()
                self._last_flush = now
            if self._f.tell() > self.max_bytes:
                self._rotate()

    def trace_config(self, model_config, cache_config) -> None:
        def plain(o):
            out = {}
            for k, v in vars(o).items():
                if k.startswith("_") or "password" in k:
                    continue
                out[k] = v if isinstance(v, (int, float, str, bool, type(None), list, tuple)) else str(v)
            return out
        self._write({"type": "CONFIG", "model_config": plain(model_config),
                     "cache_config": plain(cache_config) if cache_config is not None else None})

    def trace_request(self, kind: str, task_id: int, token_ids, slot_mapping, token_mask, namespace) -> None:
        if not self.enabled:
            return
        self._write({"type": kind, "task_id": task_id, "token_ids": _arr(token_ids),
                     "slot_mapping": _arr(slot_mapping), "token_mask": _arr(token_mask), "namespace": namespace})

    def trace_launch(self, task_ids, slot_mappings, as_batch, layerwise, counter_id) -> None:
        if not self.enabled:
            return
        self._write({"type": "LAUNCH", "task_ids": list(task_ids), "slot_mappings": [_arr(s) for s in slot_mappings],
                     "as_batch": as_batch, "layerwise_transfer": layerwise, "counter_id": counter_id})

    def trace_wait(self, task_ids, timeout, completely) -> None:
        if not self.enabled:
            return
        self._write({"type": "WAIT", "task_ids": list(task_ids), "timeout": timeout, "completely": completely})

    def trace_reset(self) -> None:
        self._write({"type": "RESET"})

    def flush(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.flush()

    def close(self) -> None:
        with self._lock:
            if self._f is not None:
                self._f.flush()
                self._f.close()
                self._f = None
