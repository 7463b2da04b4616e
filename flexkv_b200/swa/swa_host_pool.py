"""Slot allocator of the sliding-window side pool.

A slot names one page of window state in the host-side pool; the bytes live in the
storage engine's window buffer and are moved by the window worker. The allocator is a
stack free-list with double-free protection (reference: flexkv/swa/swa_host_pool.py:19-71).
"""
from __future__ import annotations

from typing import Iterable, Optional

import numpy as np

from ..common.config import SWAPoolConfig


class SWAHostPool:
    def __init__(self, config: SWAPoolConfig) -> None:
        if config.num_slots <= 0:
            raise ValueError("the window pool needs at least one slot")
        self._config = config
        self._n = int(config.num_slots)
        self._free = list(range(self._n - 1, -1, -1))
        self._is_free = np.ones(self._n, dtype=np.bool_)

    def allocate(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._is_free[s] = False
        return s

    def free(self, slot_id: int) -> None:
        s = int(slot_id)
        if s < 0 or s >= self._n:
            raise ValueError(f"invalid window slot id: {s}")
        if self._is_free[s]:
            return                      # freeing twice is harmless
        self._is_free[s] = True
        self._free.append(s)

    def free_many(self, slots: Iterable[int]) -> None:
        for s in slots:
            self.free(s)

    def reset(self) -> None:
        self._free = list(range(self._n - 1, -1, -1))
        self._is_free[:] = True

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self._n - len(self._free)

    @property
    def num_slots(self) -> int:
        return self._n

    @property
    def config(self) -> SWAPoolConfig:
        return self._config
