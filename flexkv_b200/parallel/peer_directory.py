"""Directory of prefix blocks that currently sit in some rank's GPU KV cache.

Engines publish ``block key -> (rank, gpu block)`` for the blocks of their own
prefix cache and withdraw them before the blocks are reused. A ``get`` on another
rank then pulls a matching prefix straight out of the owner's HBM over NVLink
instead of re-reading it from host memory over PCIe. Entries are leased while a
pull is in flight; a withdrawal of a leased block is deferred until the lease
ends (the same idea as the block leases of the reference's cross-node index,
csrc/dist/local_radix_tree.cpp:156-176, applied to GPU memory inside one box).
"""
from __future__ import annotations

import threading
from collections import defaultdict
from typing import Dict, List, Set, Tuple

import numpy as np


class GpuPeerDirectory:
    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._owners: Dict[int, Dict[int, int]] = defaultdict(dict)        # hash -> {rank: gpu block}
        self._by_block: Dict[Tuple[int, int], int] = {}                    # (rank, block) -> hash
        self._leases: Dict[Tuple[int, int], int] = defaultdict(int)        # (rank, block) -> pulls in flight
        self._deferred: Set[Tuple[int, int]] = set()                       # withdrawals waiting for leases
        self.stats = dict(published=0, withdrawn=0, hits=0, hit_blocks=0, deferred=0)

    def publish(self, rank: int, block_hashes: np.ndarray, gpu_blocks: np.ndarray) -> None:
        if len(block_hashes) != len(gpu_blocks):
            raise ValueError("one gpu block per block key is required")
        with self._lock:
            for h, b in zip(block_hashes.tolist(), np.asarray(gpu_blocks).tolist()):
                old = self._by_block.get((rank, b))
                if old is not None and old != h:
                    self._drop(rank, b)
                self._owners[h][rank] = b
                self._by_block[(rank, b)] = h
                self._deferred.discard((rank, b))
                self.stats["published"] += 1

    def _drop(self, rank: int, block: int) -> None:
        h = self._by_block.pop((rank, block), None)
        if h is None:
            return
        owners = self._owners.get(h)
        if owners is not None:
            owners.pop(rank, None)
            if not owners:
                del self._owners[h]
        self.stats["withdrawn"] += 1

    def withdraw_blocks(self, rank: int, gpu_blocks: np.ndarray) -> List[int]:
        """Removes the entries of these GPU blocks. Returns the blocks that are
        still being read by a peer; the caller must keep them intact until
        ``is_leased`` turns false (they are withdrawn automatically then)."""
        busy = []
        with self._lock:
            for b in np.asarray(gpu_blocks).tolist():
                if self._leases.get((rank, b), 0) > 0:
                    self._deferred.add((rank, b))
                    self.stats["deferred"] += 1
                    busy.append(b)
                else:
                    self._drop(rank, b)
        return busy

    def clear_rank(self, rank: int) -> None:
        with self._lock:
            for (r, b) in [k for k in self._by_block if k[0] == rank]:
                self._drop(r, b)

    def is_leased(self, rank: int, gpu_block: int) -> bool:
        with self._lock:
            return self._leases.get((rank, gpu_block), 0) > 0

    def match_prefix(self, block_hashes: np.ndarray, exclude_rank: int, start: int = 0, lease: bool = False
                     ) -> Tuple[int, np.ndarray, np.ndarray]:
        """Longest run ``[start, start+n)`` of keys that some other rank holds.
        Returns ``(n, owner ranks, owner gpu blocks)``; with ``lease`` the blocks
        are pinned until ``release``."""
        ranks: List[int] = []
        blocks: List[int] = []
        with self._lock:
            prefer = -1
            for h in block_hashes[start:].tolist():
                owners = self._owners.get(h)
                if not owners:
                    break
                cand = [(r, b) for r, b in owners.items()
                        if r != exclude_rank and (r, b) not in self._deferred]
                if not cand:
                    break
                # stay with the previous owner when possible: fewer, larger pulls
                pick = next(((r, b) for r, b in cand if r == prefer), cand[0])
                prefer = pick[0]
                ranks.append(pick[0])
                blocks.append(pick[1])
            if lease:
                for k in zip(ranks, blocks):
                    self._leases[k] += 1
            if ranks:
                self.stats["hits"] += 1
                self.stats["hit_blocks"] += len(ranks)
        return len(ranks), np.asarray(ranks, dtype=np.int64), np.asarray(blocks, dtype=np.int64)

    def release(self, ranks: np.ndarray, blocks: np.ndarray) -> None:
        with self._lock:
            for k in zip(np.asarray(ranks).tolist(), np.asarray(blocks).tolist()):
                n = self._leases.get(k, 0) - 1
                if n <= 0:
                    self._leases.pop(k, None)
                    if k in self._deferred:
                        self._deferred.discard(k)
                        self._drop(*k)
                else:
                    self._leases[k] = n

    def num_entries(self) -> int:
        with self._lock:
            return len(self._by_block)
