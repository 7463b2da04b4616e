"""Pure-Python prefix index: the executable specification of the native
``RadixIndex`` and its test oracle; selected at run time with
``FLEXKV_INDEX_ACCEL=0`` (reference counterpart: flexkv/cache/radixtree.py:212-943).

The class offers exactly the native interface (node handles are the node
objects themselves), so the cache engine and the tests run unchanged on either.
"""
from __future__ import annotations

import heapq
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

_U32_MAX = 0xFFFFFFFF


class PyNode:
    __slots__ = ("hashes", "blocks", "children", "parent", "ready", "lock_cnt", "hit_count", "grace_us",
                 "last_access_us", "creation_us", "live", "serial", "swa_slot", "swa_lock")

    def __init__(self, serial: int, now: int) -> None:
        self.hashes: List[int] = []
        self.blocks: List[int] = []
        self.children: Dict[int, "PyNode"] = {}
        self.parent: Optional["PyNode"] = None
        self.ready = False
        self.lock_cnt = 0
        self.hit_count = 0
        self.grace_us = self.last_access_us = self.creation_us = now
        self.live = True
        self.serial = serial
        self.swa_slot = -1          # window snapshot valid at this node's last block (-1: none)
        self.swa_lock = 0

    def size(self) -> int:
        return len(self.hashes)

    def is_leaf(self) -> bool:
        return not self.children


@dataclass
class PyMatchResult:
    num_ready_matched_blocks: int = 0
    num_matched_blocks: int = 0
    last_node_matched_length: int = 0
    last_ready_node: Optional[PyNode] = None
    last_node: Optional[PyNode] = None
    physical_blocks: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.int64))
    last_swa_node: Optional[PyNode] = None
    swa_hit_blocks: int = 0
    swa_slot: int = -1


class RadixTreeIndex:
    def __init__(self, tokens_per_block: int, max_num_blocks: int = 0, eviction_policy: str = "lru",
                 hit_reward_seconds: float = 0.0, slru_threshold: int = 2) -> None:
        if tokens_per_block <= 0 or tokens_per_block & (tokens_per_block - 1):
            raise ValueError("tokens_per_block must be a power of two")
        self.tokens_per_block = tokens_per_block
        self.max_num_blocks = max_num_blocks
        self.policy = eviction_policy.lower()
        if self.policy not in ("lru", "lfu", "fifo", "mru", "filo", "slru"):
            raise ValueError(f"unknown eviction policy: {eviction_policy}")
        self.hit_reward_us = int(hit_reward_seconds * 1e6)
        self.slru_threshold = slru_threshold
        self._clock_override = -1
        self._serial = 0
        self._total_blocks = 0
        self._nodes = 0
        self._root = self._new_node()
        self._root.ready = True
        self._stats = dict(hit=0, match=0, miss=0, insert_blocks=0, evict_blocks=0)
        self._swa_lru: List[PyNode] = []       # least recently used first
        self._swa_armed = False                # a snapshot was mounted at least once
        self._freed_swa: List[int] = []

    # ---- helpers ----------------------------------------------------------------
    def _now(self) -> int:
        return self._clock_override if self._clock_override >= 0 else int(time.time() * 1e6)

    def _new_node(self) -> PyNode:
        self._serial += 1
        self._nodes += 1
        return PyNode(self._serial, self._now())

    def _free(self, n: PyNode) -> None:
        self._drop_swa(n)
        n.live = False
        n.children = {}
        self._nodes -= 1

    def _touch(self, n: PyNode, now: int) -> None:
        n.last_access_us = now
        n.grace_us = max(n.grace_us, now) + self.hit_reward_us
        if n.hit_count < _U32_MAX:
            n.hit_count += 1

    def _check(self, h: Optional[PyNode]) -> PyNode:
        if h is None or not h.live:
            raise RuntimeError("radix index: stale or null node handle")
        return h

    # ---- queries ----------------------------------------------------------------
    def match_prefix(self, block_hashes: np.ndarray, num_blocks: int = -1,
                     update_cache_info: bool = True) -> PyMatchResult:
        hashes = block_hashes
        n = len(hashes) if num_blocks < 0 or num_blocks > len(hashes) else num_blocks
        r = PyMatchResult(last_node=self._root, last_ready_node=self._root)
        blocks: List[int] = []
        now = self._now() if update_cache_info else 0
        cur, prefix, ready_chain = self._root, 0, True
        while prefix < n:
            c = cur.children.get(int(hashes[prefix]))
            if c is None:
                break
            span = min(c.size(), n - prefix)
            if c.hashes[span - 1] == int(hashes[prefix + span - 1]):
                m = span
            else:
                lo, hi = 1, span - 1
                while lo < hi:
                    mid = (lo + hi + 1) >> 1
                    if c.hashes[mid - 1] == int(hashes[prefix + mid - 1]):
                        lo = mid
                    else:
                        hi = mid - 1
                m = lo
            if update_cache_info:
                self._touch(c, now)
            blocks.extend(c.blocks[:m])
            prefix += m
            r.last_node, r.last_node_matched_length = c, m
            if ready_chain and c.ready:
                r.num_ready_matched_blocks, r.last_ready_node = prefix, c
                if c.swa_slot >= 0 and m == c.size():      # only a fully matched node exposes its snapshot
                    r.last_swa_node, r.swa_hit_blocks, r.swa_slot = c, prefix, c.swa_slot
                    if update_cache_info:
                        self._swa_touch(c)
            else:
                ready_chain = False
            if m < c.size():
                break
            cur = c
        r.num_matched_blocks = prefix
        r.physical_blocks = np.asarray(blocks, dtype=np.int64)
        if n > 0:
            self._stats["hit" if prefix == n else "match" if prefix > 0 else "miss"] += 1
        return r

    # ---- mutation ---------------------------------------------------------------
    def _split(self, node: PyNode, k: int) -> PyNode:
        pre = self._new_node()
        parent = node.parent
        old_head = node.hashes[0]
        pre.hashes, pre.blocks = node.hashes[:k], node.blocks[:k]
        node.hashes, node.blocks = node.hashes[k:], node.blocks[k:]
        pre.ready, pre.hit_count = node.ready, node.hit_count
        pre.grace_us, pre.last_access_us, pre.creation_us = node.grace_us, node.last_access_us, node.creation_us
        pre.parent = parent
        parent.children[old_head] = pre
        pre.children = {node.hashes[0]: node}
        node.parent = pre
        return pre

    def _validate(self, hashes, n: int, num_insert: int, m: PyMatchResult) -> None:
        def stale(why: str):
            raise RuntimeError(f"radix index insert: stale match result; rematch ({why})")
        node = m.last_node
        if node is None or not node.live:
            stale("node no longer exists")
        if m.num_matched_blocks < 0 or m.num_matched_blocks > n:
            stale("matched length out of range")
        if node is self._root:
            if m.num_matched_blocks != 0:
                stale("root cannot carry a match")
            if num_insert > 0 and int(hashes[0]) in node.children:
                stale("first block appeared meanwhile")
            return
        ml = m.last_node_matched_length
        if ml <= 0 or ml > node.size() or ml > m.num_matched_blocks:
            stale("matched span out of range")
        if node.parent is None or node.parent.children.get(node.hashes[0]) is not node:
            stale("node not under its parent")
        if node.hashes[ml - 1] != int(hashes[m.num_matched_blocks - 1]) or \
                node.hashes[0] != int(hashes[m.num_matched_blocks - ml]):
            stale("matched span changed")
        if num_insert > m.num_matched_blocks:
            if ml < node.size():
                if node.hashes[ml] == int(hashes[m.num_matched_blocks]):
                    stale("split point does not diverge")
            elif int(hashes[m.num_matched_blocks]) in node.children:
                stale("target child exists")

    def insert(self, physical_block_ids: np.ndarray, block_hashes: np.ndarray, num_insert_blocks: int = -1,
               is_ready: bool = True, match_result: Optional[PyMatchResult] = None) -> Optional[PyNode]:
        n = len(block_hashes)
        num_insert = n if num_insert_blocks < 0 else num_insert_blocks
        if num_insert > n:
            raise ValueError("radix index insert: num_insert exceeds hash count")
        m = match_result if match_result is not None else self.match_prefix(block_hashes, num_insert, False)
        if num_insert <= m.num_matched_blocks:
            return None
        if len(physical_block_ids) != num_insert - m.num_matched_blocks:
            raise ValueError("radix index insert: physical block count != num_insert - num_matched")
        self._validate(block_hashes, n, num_insert, m)
        if self.max_num_blocks > 0 and self._total_blocks + len(physical_block_ids) > self.max_num_blocks:
            raise RuntimeError("radix index insert: capacity exceeded")
        parent = m.last_node
        if parent is not self._root and m.last_node_matched_length < parent.size():
            parent = self._split(parent, m.last_node_matched_length)
        node = self._new_node()
        node.hashes = [int(h) for h in block_hashes[m.num_matched_blocks:num_insert]]
        node.blocks = [int(b) for b in physical_block_ids]
        node.ready = is_ready
        node.parent = parent
        parent.children[node.hashes[0]] = node
        self._total_blocks += len(node.blocks)
        self._stats["insert_blocks"] += len(node.blocks)
        return node

    def _evictable(self, n: PyNode) -> bool:
        return n is not self._root and n.live and n.is_leaf() and n.lock_cnt == 0 and n.ready

    def _key(self, n: PyNode) -> Tuple:
        p = self.policy
        if p == "lru":
            k: Tuple = (n.grace_us,)
        elif p == "mru":
            k = (-n.grace_us,)
        elif p == "fifo":
            k = (n.creation_us,)
        elif p == "filo":
            k = (-n.creation_us,)
        elif p == "lfu":
            k = (n.hit_count, n.last_access_us)
        else:
            k = (1 if n.hit_count >= self.slru_threshold else 0, n.last_access_us)
        return k + (n.serial,)

    def _leaves(self) -> List[PyNode]:
        out, stack = [], [self._root]
        while stack:
            x = stack.pop()
            if x.children:
                stack.extend(x.children.values())
            elif x is not self._root:
                out.append(x)
        return out

    def evict(self, num_blocks: int) -> Tuple[np.ndarray, np.ndarray]:
        blocks: List[int] = []
        hashes: List[int] = []
        if num_blocks > 0:
            heap = [(self._key(l), id(l), l) for l in self._leaves() if self._evictable(l)]
            heapq.heapify(heap)
            need = num_blocks
            while need > 0 and heap:
                _, _, node = heapq.heappop(heap)
                sz = node.size()
                if sz > need:
                    self._drop_swa(node)        # the snapshot described the dropped tail
                    blocks.extend(node.blocks[sz - need:])
                    hashes.extend(node.hashes[sz - need:])
                    node.blocks, node.hashes = node.blocks[:sz - need], node.hashes[:sz - need]
                    self._total_blocks -= need
                    need = 0
                    break
                blocks.extend(node.blocks)
                hashes.extend(node.hashes)
                self._total_blocks -= sz
                need -= sz
                parent = node.parent
                del parent.children[node.hashes[0]]
                self._free(node)
                parent = self._prune_snapshotless_leaves(parent, blocks, hashes)
                if self._evictable(parent):
                    heapq.heappush(heap, (self._key(parent), id(parent), parent))
        self._stats["evict_blocks"] += len(blocks)
        return np.asarray(blocks, dtype=np.int64), np.asarray(hashes, dtype=np.uint64)

    def _prune_snapshotless_leaves(self, node: PyNode, blocks: List[int], hashes: List[int]) -> PyNode:
        """Once window snapshots are in use, a leaf without one serves no window-aware request: after a
        deletion the ancestors that became such leaves (evictable, no snapshot) go too, their blocks are
        appended beyond what the caller asked for. Returns the first ancestor that stays
        (reference: flexkv/cache/radixtree.py:726-749)."""
        if not self._swa_armed:
            return node
        while node is not self._root and node.is_leaf() and node.swa_slot < 0 and self._evictable(node):
            blocks.extend(node.blocks)
            hashes.extend(node.hashes)
            self._total_blocks -= node.size()
            parent = node.parent
            del parent.children[node.hashes[0]]
            self._free(node)
            node = parent
        return node

    def lock(self, h: PyNode) -> None:
        self._check(h).lock_cnt += 1

    def unlock(self, h: PyNode) -> None:
        n = self._check(h)
        if n.lock_cnt <= 0:
            raise RuntimeError("radix index: unlock of an unlocked node")
        n.lock_cnt -= 1

    def set_ready(self, node: PyNode, ready: bool = True, ready_length: int = -1) -> None:
        n = self._check(node)
        covered = 0
        while n is not None and n is not self._root:
            n.ready = ready
            covered += n.size()
            if ready_length < 0 or covered >= ready_length:
                break
            n = n.parent

    def remove_unready_leaf(self, h: Optional[PyNode]) -> np.ndarray:
        if h is None or not h.live or h is self._root or not h.is_leaf() or h.ready or h.lock_cnt > 0:
            return np.zeros(0, dtype=np.int64)
        out = np.asarray(h.blocks, dtype=np.int64)
        self._total_blocks -= h.size()
        del h.parent.children[h.hashes[0]]
        self._free(h)
        return out

    def truncate_unready_leaf(self, h: Optional[PyNode], keep: int) -> np.ndarray:
        if keep <= 0:
            return self.remove_unready_leaf(h)
        if h is None or not h.live or h is self._root or not h.is_leaf() or h.ready or h.lock_cnt > 0 \
                or keep >= h.size():
            return np.zeros(0, dtype=np.int64)
        out = np.asarray(h.blocks[keep:], dtype=np.int64)
        h.blocks, h.hashes = h.blocks[:keep], h.hashes[:keep]
        self._total_blocks -= len(out)
        return out

    def reset(self) -> np.ndarray:
        all_blocks: List[int] = []
        stack = list(self._root.children.values())
        while stack:
            x = stack.pop()
            stack.extend(x.children.values())
            all_blocks.extend(x.blocks)
            self._free(x)
        self._root.children = {}
        self._total_blocks = 0
        self._swa_lru, self._freed_swa = [], []
        return np.asarray(all_blocks, dtype=np.int64)

    # ---- warm restart (same image as the native index) -------------------------------------
    def export_ready(self):
        """Flat pre-order image of the ready nodes: ``(parents, sizes, hashes, blocks)``; node ``i``
        hangs below ``parents[i]`` (-1 = root). Subtrees below an unready node are left out."""
        parents: List[int] = []
        sizes: List[int] = []
        hashes: List[int] = []
        blocks: List[int] = []
        stack = [(c, -1) for _, c in sorted(self._root.children.items(), reverse=True)]
        while stack:
            n, parent_pos = stack.pop()
            if not n.live or not n.ready:
                continue
            pos = len(parents)
            parents.append(parent_pos)
            sizes.append(n.size())
            hashes.extend(n.hashes)
            blocks.extend(n.blocks)
            stack.extend((c, pos) for _, c in sorted(n.children.items(), reverse=True))
        return (np.asarray(parents, dtype=np.int32), np.asarray(sizes, dtype=np.int64),
                np.asarray(hashes, dtype=np.uint64), np.asarray(blocks, dtype=np.int64))

    def import_snapshot(self, parents, sizes, hashes, blocks) -> int:
        """Rebuilds an exported image in an empty index; returns the number of blocks restored.
        A malformed image raises ValueError and leaves the index empty."""
        if not self.is_empty():
            raise ValueError("radix index import: the index is not empty")
        parents = np.asarray(parents, dtype=np.int64)
        sizes = np.asarray(sizes, dtype=np.int64)
        hashes = np.asarray(hashes, dtype=np.uint64)
        blocks = np.asarray(blocks, dtype=np.int64)
        nn = len(parents)
        if len(sizes) != nn:
            raise ValueError("radix index import: parents / sizes differ in length")
        if nn and (sizes.min() <= 0 or (parents < -1).any() or (parents >= np.arange(nn)).any()):
            raise ValueError("radix index import: empty node or a node listed before its parent")
        total = int(sizes.sum())
        if len(hashes) != total or len(blocks) != total:
            raise ValueError("radix index import: hashes / blocks do not cover the nodes")
        if self.max_num_blocks > 0 and total > self.max_num_blocks:
            raise ValueError("radix index import: more blocks than this index may hold")
        if total and (blocks.min() < 0 or (self.max_num_blocks > 0 and blocks.max() >= self.max_num_blocks)):
            raise ValueError("radix index import: block id out of range")
        if np.unique(blocks).size != total:
            raise ValueError("radix index import: a block id is listed twice")
        off = np.concatenate([[0], np.cumsum(sizes)])
        path: List[int] = []
        open_: List[Tuple[int, int]] = []
        try:
            for i in range(nn):
                while open_ and open_[-1][0] != parents[i]:
                    open_.pop()
                if not open_ and parents[i] != -1:
                    raise ValueError("radix index import: the image is not in pre-order")
                del path[open_[-1][1] if open_ else 0:]
                path.extend(hashes[off[i]:off[i + 1]].tolist())
                h = self.insert(blocks[off[i]:off[i + 1]], np.asarray(path, dtype=np.uint64), len(path), True, None)
                if h is None:
                    raise ValueError("radix index import: two nodes share a path")
                open_.append((i, len(path)))
        except Exception:
            self.reset()
            raise
        return total

    # ---- window snapshots mounted on nodes (same rules as the native index) ---------------
    def _drop_swa(self, n: PyNode) -> None:
        if n.swa_slot >= 0:
            self._freed_swa.append(n.swa_slot)
            self._swa_lru = [x for x in self._swa_lru if x is not n]
        n.swa_slot, n.swa_lock = -1, 0

    def _swa_touch(self, n: PyNode) -> None:
        self._swa_lru = [x for x in self._swa_lru if x is not n]
        self._swa_lru.append(n)

    def set_swa(self, h: PyNode, slot: int) -> None:
        n = self._check(h)
        if n is self._root:
            raise ValueError("radix index: the root carries no window snapshot")
        if slot < 0:
            raise ValueError("radix index: negative snapshot slot")
        if n.swa_slot >= 0 and n.swa_slot != slot:
            self._freed_swa.append(n.swa_slot)
        n.swa_slot = int(slot)
        self._swa_armed = True          # stays set across reset(): the deployment uses window snapshots
        self._swa_touch(n)

    def has_swa(self, h) -> bool:
        return h is not None and h.live and h is not self._root and h.swa_slot >= 0

    def swa_slot(self, h) -> int:
        return self._check(h).swa_slot

    def swa_lock_cnt(self, h) -> int:
        return self._check(h).swa_lock

    def lock_swa(self, h) -> None:
        n = self._check(h)
        if n.swa_slot < 0:
            raise RuntimeError("radix index: node has no window snapshot to lock")
        n.lock_cnt += 1
        n.swa_lock += 1

    def unlock_swa(self, h) -> None:
        if h is None or not h.live:
            return
        if h.swa_lock > 0:
            h.swa_lock -= 1
        if h.lock_cnt > 0:
            h.lock_cnt -= 1

    def evict_swa(self, n: int):
        blocks: List[int] = []
        hashes: List[int] = []
        freed = 0
        for node in list(self._swa_lru):
            if freed >= n:
                break
            if node.swa_lock > 0:
                continue
            if node.is_leaf() and node.lock_cnt == 0 and node.ready:
                blocks.extend(node.blocks)
                hashes.extend(node.hashes)
                self._total_blocks -= node.size()
                self._stats["evict_blocks"] += node.size()
                parent = node.parent
                del parent.children[node.hashes[0]]
                self._free(node)
                before = len(blocks)
                self._prune_snapshotless_leaves(parent, blocks, hashes)
                self._stats["evict_blocks"] += len(blocks) - before
            else:
                self._drop_swa(node)
            freed += 1
        return np.asarray(blocks, dtype=np.int64), np.asarray(hashes, dtype=np.uint64), freed

    def drain_freed_swa_slots(self) -> np.ndarray:
        out, self._freed_swa = self._freed_swa, []
        return np.asarray(out, dtype=np.int32)

    def total_swa_slots(self) -> int:
        return len(self._swa_lru)

    # ---- introspection (mirrors the native class) -------------------------------------
    def alive(self, h) -> bool:
        return h is not None and h.live

    def is_root(self, h) -> bool:
        return h is self._root

    def root(self) -> PyNode:
        return self._root

    def node_size(self, h) -> int:
        return self._check(h).size()

    def node_ready(self, h) -> bool:
        return self._check(h).ready

    def node_lock_cnt(self, h) -> int:
        return self._check(h).lock_cnt

    def node_parent(self, h):
        return self._check(h).parent

    def node_is_leaf(self, h) -> bool:
        return self._check(h).is_leaf()

    def node_hit_count(self, h) -> int:
        return self._check(h).hit_count

    def total_cached_blocks(self) -> int:
        return self._total_blocks

    def total_ready_blocks(self) -> int:
        t, stack = 0, list(self._root.children.values())
        while stack:
            x = stack.pop()
            stack.extend(x.children.values())
            if x.ready:
                t += x.size()
        return t

    def num_nodes(self) -> int:
        return self._nodes

    def num_leaves(self) -> int:
        return len(self._leaves())

    def num_evictable_blocks(self) -> int:
        def walk(n: PyNode) -> Tuple[bool, int]:
            good = n is not self._root and n.lock_cnt == 0 and n.ready
            total = 0
            for c in n.children.values():
                g, t = walk(c)
                good = good and g
                total += t
            if good:
                total += n.size()
            return good, total
        return walk(self._root)[1]

    def is_empty(self) -> bool:
        return not self._root.children

    def set_clock_override(self, us: int) -> None:
        self._clock_override = us

    def set_policy(self, p: str) -> None:
        self.policy = p.lower()

    def stats(self) -> Dict[str, int]:
        return dict(self._stats)
