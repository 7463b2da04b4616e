"""Block id pool of one tier. The numpy implementation is the executable
specification; ``Mempool(..., native=True)`` uses the C++ pool with the same
checks (duplicate ids, double free, range) — flexkv/cache/mempool.py:26-56."""
from __future__ import annotations

import numpy as np

from .. import _native


class NotEnoughSpaceError(RuntimeError):
    pass


class Mempool:
    def __init__(self, num_total_blocks: int, native: bool = True) -> None:
        if num_total_blocks < 0:
            raise ValueError("num_total_blocks must be non-negative")
        self.num_total_blocks = int(num_total_blocks)
        self._native = _native.C.BlockPool(self.num_total_blocks) if native else None
        if self._native is None:
            self._free_mask = np.ones(self.num_total_blocks, dtype=np.bool_)
            self._num_free = self.num_total_blocks

    def reset(self) -> None:
        if self._native is not None:
            self._native.reset()
        else:
            self._free_mask[:] = True
            self._num_free = self.num_total_blocks

    def allocate_blocks(self, num: int, strict: bool = True) -> np.ndarray:
        if num < 0:
            raise ValueError("num must be non-negative")
        if self._native is not None:
            try:
                return self._native.allocate(int(num), strict)
            except RuntimeError as e:
                raise NotEnoughSpaceError(str(e)) from None
        if num > self._num_free:
            if strict:
                raise NotEnoughSpaceError(f"need {num} blocks, {self._num_free} free")
            num = self._num_free
        ids = np.flatnonzero(self._free_mask)[:num].astype(np.int64)
        self._free_mask[ids] = False
        self._num_free -= int(ids.size)
        return ids

    def recycle_blocks(self, block_ids: np.ndarray) -> None:
        block_ids = np.ascontiguousarray(block_ids, dtype=np.int64)
        if block_ids.size == 0:
            return
        if self._native is not None:
            self._native.recycle(block_ids)
            return
        if block_ids.min() < 0 or block_ids.max() >= self.num_total_blocks:
            raise IndexError("block id out of range")
        if np.unique(block_ids).size != block_ids.size:
            raise RuntimeError("duplicate block ids in recycle")
        if self._free_mask[block_ids].any():
            raise RuntimeError("double free")
        self._free_mask[block_ids] = True
        self._num_free += int(block_ids.size)

    def reserve_blocks(self, block_ids: np.ndarray) -> None:
        """Takes these specific free blocks out of the pool (blocks of an index mounted from disk)."""
        block_ids = np.ascontiguousarray(block_ids, dtype=np.int64)
        if block_ids.size == 0:
            return
        if self._native is not None:
            self._native.reserve(block_ids)
            return
        if block_ids.min() < 0 or block_ids.max() >= self.num_total_blocks:
            raise IndexError("block id out of range")
        if np.unique(block_ids).size != block_ids.size or not self._free_mask[block_ids].all():
            raise RuntimeError("block already in use or listed twice")
        self._free_mask[block_ids] = False
        self._num_free -= int(block_ids.size)

    @property
    def num_free_blocks(self) -> int:
        return self._native.num_free if self._native is not None else self._num_free

    @property
    def num_used_blocks(self) -> int:
        return self.num_total_blocks - self.num_free_blocks
