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
