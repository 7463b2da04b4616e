"""KV events for Dynamo-style routers: "stored" when blocks enter a tier's index,
"removed" when they are evicted (flexkv/integration/dynamo/collector.py:18-116)."""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Any, Callable, List, Optional

import numpy as np

from ...common.transfer import DeviceType


@dataclass
class KVEvent:
    kind: str                  # "stored" | "removed"
    device: str
    block_hashes: List[int]
    event_id: int = 0


class KVEventCollector:
    def __init__(self, publisher: Optional[Callable[[KVEvent], None]] = None, max_buffer: int = 65536) -> None:
        self._publisher = publisher
        self._buf: List[KVEvent] = []
        self._lock = threading.Lock()
        self._next = 0
        self._max = max_buffer

    def attach(self, global_cache_engine: Any) -> None:
        global_cache_engine.event_listeners.append(self)
        for eng in global_cache_engine.cache_engines.values():
            eng.on_insert.append(lambda dev, blocks, hashes: self.publish_stored(dev, hashes))

    def _emit(self, kind: str, device: DeviceType, hashes: np.ndarray) -> None:
        if len(hashes) == 0:
            return
        with self._lock:
            ev = KVEvent(kind, device.name, [int(h) for h in hashes], self._next)
            self._next += 1
            if self._publisher is not None:
                self._publisher(ev)
            else:
                self._buf.append(ev)
                del self._buf[:-self._max]

    def publish_stored(self, device: DeviceType, hashes: np.ndarray) -> None:
        self._emit("stored", device, hashes)

    def publish_removed(self, device: DeviceType, hashes: np.ndarray) -> None:
        self._emit("removed", device, hashes)

    def take_events(self) -> List[KVEvent]:
        with self._lock:
            out, self._buf = self._buf, []
            return out

    def close(self) -> None:
        """Nothing runs in the background here (events are buffered by the caller's thread); kept for callers
        written against the reference, whose collector owns a worker thread."""


def to_vllm_events(events: List[KVEvent], block_size: int) -> List[Any]:
    """The same events as vLLM's own ``BlockStored`` / ``BlockRemoved`` records, which is what the engine's event
    publisher serialises (flexkv/integration/dynamo/collector.py:56-82). Fields that newer engine versions added
    keep their defaults. Without vLLM the events come back unchanged."""
    try:
        from vllm.distributed.kv_events import BlockRemoved, BlockStored
    except Exception:  # noqa: BLE001 - no engine in this process
        return list(events)
    out: List[Any] = []
    stored_fields = set(getattr(BlockStored, "__struct_fields__", ()))
    for ev in events:
        if ev.kind == "stored":
            kw = dict(block_hashes=list(ev.block_hashes), parent_block_hash=None, token_ids=[], block_size=int(block_size),
                      lora_id=None, medium=ev.device, lora_name=None)
            out.append(BlockStored(**{k: v for k, v in kw.items() if not stored_fields or k in stored_fields}))
        else:
            out.append(BlockRemoved(block_hashes=list(ev.block_hashes), medium=ev.device))
    return out
