"""Control plane: per-tier prefix caches and the planner that turns a get/put
request into a transfer graph.

Behavioural counterpart of the reference's ``CacheEngine`` /
``GlobalCacheEngine`` (flexkv/cache/cache_engine.py:272-867 tier engine,
:1109-1232 get, :1718-1997 local get plan, :2000-2081 put, :2488-2701 local put
plan, :2919-3020 completion / abort, :480-582 take with eviction). The tiers
are inclusive and write-through: a put lands in the host pool and, when
enabled, on SSD; evicting from one tier never writes back to another.
"""
from __future__ import annotations

import logging
import math
import os
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np

from .. import _native
from ..common.block import SequenceMeta
from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from ..common.debug import EvictionLogAggregator, log_op
from ..common.transfer import DeviceType, TransferOp, TransferOpGraph, TransferType
from . import persist
from .mempool import Mempool, NotEnoughSpaceError
from .radixtree import RadixTreeIndex

_EMPTY = np.zeros(0, dtype=np.int64)


def slot_mapping_to_block_ids(slot_mapping: np.ndarray, tokens_per_block: int) -> np.ndarray:
    """One GPU block id per block: the engine's flat token slot is
    ``block_id * tokens_per_block + offset`` (flexkv/cache/cache_engine.py:3338-3340)."""
    return np.ascontiguousarray(slot_mapping[::tokens_per_block] // tokens_per_block, dtype=np.int64)


class CacheEngine:
    """Prefix index + block pool of one tier."""

    def __init__(self, device_type: DeviceType, num_total_blocks: int, tokens_per_block: int,
                 evict_ratio: float = 0.0, hit_reward_seconds: float = 0.0, eviction_policy: str = "lru",
                 slru_threshold: int = 2, evict_start_threshold: float = 1.0,
                 accel: Optional[bool] = None) -> None:
        if num_total_blocks <= 0:
            raise ValueError(f"invalid num_total_blocks: {num_total_blocks}")
        if tokens_per_block <= 0 or tokens_per_block & (tokens_per_block - 1):
            raise ValueError(f"tokens_per_block must be a power of two, got {tokens_per_block}")
        if not 0.0 <= evict_ratio <= 1.0:
            raise ValueError("evict_ratio must be in [0, 1]")
        if not 0.0 < evict_start_threshold <= 1.0:
            raise ValueError("evict_start_threshold must be in (0, 1]")
        self.device_type = device_type
        self.num_total_blocks = int(num_total_blocks)
        self.tokens_per_block = tokens_per_block
        self.evict_ratio = evict_ratio
        self.evict_start_threshold = evict_start_threshold
        self.accel = GLOBAL_CONFIG_FROM_ENV.index_accel if accel is None else accel
        if self.accel:
            self.index = _native.C.RadixIndex(tokens_per_block, self.num_total_blocks, eviction_policy,
                                              float(hit_reward_seconds), int(slru_threshold))
        else:
            self.index = RadixTreeIndex(tokens_per_block, self.num_total_blocks, eviction_policy,
                                        float(hit_reward_seconds), int(slru_threshold))
        self.mempool = Mempool(self.num_total_blocks, native=self.accel)
        self.on_evict: List[Callable[[DeviceType, np.ndarray, np.ndarray], None]] = []
        self.on_insert: List[Callable[[DeviceType, np.ndarray, np.ndarray], None]] = []
        self.num_evicted_total = 0

    def reset(self) -> None:
        self.index.reset()
        self.mempool.reset()
        if self.swa_pool is not None:
            self.swa_pool.reset()

    # ---- sliding-window snapshots (node-mounted; native index only) ---------------------
    swa_pool = None

    @property
    def swa_enabled(self) -> bool:
        return self.swa_pool is not None

    def attach_swa(self, pool) -> None:
        if not hasattr(self.index, "set_swa"):
            raise ValueError("window snapshots need the native index (FLEXKV_INDEX_ACCEL=1)")
        self.swa_pool = pool

    def _drain_swa(self) -> None:
        if self.swa_pool is not None:
            self.swa_pool.free_many(self.index.drain_freed_swa_slots().tolist())

    def alloc_swa_slot(self) -> Optional[int]:
        """A free window slot, evicting least-recently-used snapshots when the pool is full
        (unlocked leaves that only a snapshot keeps alive go with their blocks)."""
        if self.swa_pool is None:
            return None
        self._drain_swa()
        slot = self.swa_pool.allocate()
        if slot is not None:
            return slot
        want = max(1, int(self.swa_pool.num_slots * self.swa_pool.config.evict_ratio))
        blocks, hashes, _ = self.index.evict_swa(want)
        if len(blocks):
            self.mempool.recycle_blocks(blocks)
            self.num_evicted_total += int(len(blocks))
            for cb in self.on_evict:
                cb(self.device_type, blocks, hashes)
        self._drain_swa()
        return self.swa_pool.allocate()

    def mount_swa(self, node, slot: int) -> bool:
        """Attaches the snapshot in ``slot`` to ``node`` (valid at its last block)."""
        if node is None or not self.index.alive(node) or self.index.is_root(node):
            self.swa_pool.free(slot)
            return False
        self.index.set_swa(node, int(slot))
        self._drain_swa()               # a replaced snapshot returns its slot
        return True

    def match(self, seq: SequenceMeta, update_cache_info: bool = True):
        return self.index.match_prefix(seq.block_hashes, seq.num_blocks, update_cache_info)

    def insert(self, seq: SequenceMeta, physical_block_ids: np.ndarray, num_insert_blocks: int = -1,
               is_ready: bool = True, match_result: Any = None):
        node = self.index.insert(np.ascontiguousarray(physical_block_ids, dtype=np.int64), seq.block_hashes,
                                 num_insert_blocks, is_ready, match_result)
        if node is not None and self.on_insert:
            n = len(physical_block_ids)
            end = seq.num_blocks if num_insert_blocks < 0 else num_insert_blocks
            for cb in self.on_insert:
                cb(self.device_type, np.asarray(physical_block_ids), seq.block_hashes[end - n:end])
        return node

    def lock_node(self, node) -> None:
        self.index.lock(node)

    def unlock(self, node) -> None:
        if self.index.alive(node):
            self.index.unlock(node)

    def set_ready(self, node, ready: bool = True, ready_length: int = -1) -> None:
        if self.index.alive(node):
            self.index.set_ready(node, ready, ready_length)

    def rollback_unready_insert(self, node) -> int:
        """Drops a node inserted by a plan that never produced its data; its
        blocks go back to the pool. Returns the number of blocks released."""
        if node is None or not self.index.alive(node):
            return 0
        blocks = self.index.remove_unready_leaf(node)
        if len(blocks):
            self.mempool.recycle_blocks(blocks)
        return int(len(blocks))

    def take(self, num_required_blocks: int, protected_node=None, strict: bool = True) -> np.ndarray:
        """Allocates blocks, evicting when the pool is short or past the
        configured utilisation (flexkv/cache/cache_engine.py:480-582)."""
        n = int(num_required_blocks)
        if n <= 0:
            return _EMPTY
        total, free = self.num_total_blocks, self.mempool.num_free_blocks
        used = total - free
        over = used / total >= self.evict_start_threshold and self.evict_start_threshold < 1.0
        if n > free or over:
            to_threshold = max(0, used + n - int(math.floor(total * self.evict_start_threshold)))
            amount = max(n - free, to_threshold, int(total * self.evict_ratio))
            if amount > 0:
                locked = protected_node is not None and self.index.alive(protected_node) \
                    and not self.index.is_root(protected_node)
                if locked:
                    self.index.lock(protected_node)
                try:
                    blocks, hashes = self.index.evict(amount)
                finally:
                    if locked:
                        self.index.unlock(protected_node)
                if len(blocks):
                    self.mempool.recycle_blocks(blocks)
                    self.num_evicted_total += int(len(blocks))
                    for cb in self.on_evict:
                        cb(self.device_type, blocks, hashes)
                    self._drain_swa()
        if n > self.mempool.num_free_blocks:
            # the eviction could not make room (everything left is locked, unready or leased): say so at once, the
            # caller is about to skip an offload or fail a restore (reference: tests/test_operational_logging.py:63-77)
            log_op("eviction", "batch", "target_miss", level=logging.WARNING, tier=self.device_type.name, wanted=n,
                   free=self.mempool.num_free_blocks, total=self.num_total_blocks, target_met="false")
        if n > self.mempool.num_free_blocks and strict:
            raise NotEnoughSpaceError(f"{self.device_type.name}: need {n} blocks, "
                                      f"{self.mempool.num_free_blocks} free after eviction")
        return self.mempool.allocate_blocks(min(n, self.mempool.num_free_blocks), strict=False)

    def recycle(self, block_ids: np.ndarray) -> None:
        if block_ids is not None and len(block_ids):
            self.mempool.recycle_blocks(block_ids)


class TransferPlanHandle:
    """Exactly one of ``complete`` / ``abort`` runs, once
    (flexkv/cache/cache_engine.py:236-264)."""

    def __init__(self, complete: Callable[[], None], abort: Callable[[], None]) -> None:
        self._complete, self._abort = complete, abort
        self._done = False
        self._lock = threading.Lock()

    def _once(self) -> bool:
        with self._lock:
            if self._done:
                return False
            self._done = True
            return True

    def complete(self) -> None:
        if self._once():
            self._complete()

    def abort(self) -> None:
        if self._once():
            self._abort()

    def __call__(self) -> None:
        self.complete()

    @property
    def finished(self) -> bool:
        return self._done


@dataclass
class TransferPlan:
    graph: TransferOpGraph
    finished_ops_ids: List[int] = field(default_factory=list)
    # device -> list of (node, ready_length); ready_length 0 = lock only
    nodes: Dict[DeviceType, List[Tuple[Any, int]]] = field(default_factory=dict)
    inserted: Dict[DeviceType, List[Any]] = field(default_factory=dict)   # rollback candidates
    buffer_to_free: Dict[DeviceType, np.ndarray] = field(default_factory=dict)
    op_callback_dict: Dict[int, Callable] = field(default_factory=dict)
    num_gpu_blocks_to_transfer: int = 0
    skipped_gpu_blocks: int = 0
    peer_leases: Optional[Tuple[np.ndarray, np.ndarray]] = None   # (ranks, gpu blocks) pinned in the peer directory
    swa_locked: List[Any] = field(default_factory=list)            # (tier engine, node) pairs this plan window-locked
    swa_pending: Dict[int, int] = field(default_factory=dict)      # side op id -> host slot not yet mounted
    swa_pending_tier: Dict[int, Any] = field(default_factory=dict)  # side op id -> (tier engine, its slot) not yet mounted
    partial_blocks: Optional[int] = None                           # prefetch: blocks (from bstart) that really arrived


def _block_range(token_mask: np.ndarray, tokens_per_block: int) -> Tuple[int, int]:
    idx = np.flatnonzero(token_mask)
    if idx.size == 0:
        return 0, 0
    return int(idx[0]) // tokens_per_block, int(idx[-1]) // tokens_per_block + 1


class GlobalCacheEngine:
    _index_saved = False

    def __init__(self, cache_config: CacheConfig, model_config: ModelConfig) -> None:
        self.cache_config = cache_config
        self.model_config = model_config
        self.tokens_per_block = cache_config.tokens_per_block
        self._cache_tree_lock = threading.RLock()
        env = GLOBAL_CONFIG_FROM_ENV
        policy = cache_config.eviction_policy or env.eviction_policy
        common = dict(tokens_per_block=self.tokens_per_block, evict_ratio=env.evict_ratio,
                      hit_reward_seconds=env.hit_reward_seconds, eviction_policy=policy,
                      slru_threshold=env.slru_protected_threshold, evict_start_threshold=env.evict_start_threshold)
        self.cache_engines: Dict[DeviceType, CacheEngine] = {}
        self.cpu_cache_engine: Optional[CacheEngine] = None
        self.ssd_cache_engine: Optional[CacheEngine] = None
        self.remote_cache_engine: Optional[CacheEngine] = None
        self.node_registry = None
        if cache_config.enable_cpu and cache_config.enable_p2p_cpu:
            # host blocks are published to the other nodes of the registry and theirs can be pulled
            from .hie_cache_engine import HierarchyLRCacheEngine, get_node_registry
            self.node_registry = get_node_registry(cache_config, model_config)
            self.cpu_cache_engine = HierarchyLRCacheEngine(DeviceType.CPU, cache_config.num_cpu_blocks,
                                                           registry=self.node_registry, **common)
            self.cache_engines[DeviceType.CPU] = self.cpu_cache_engine
        elif cache_config.enable_cpu:
            self.cpu_cache_engine = CacheEngine(DeviceType.CPU, cache_config.num_cpu_blocks, **common)
            self.cache_engines[DeviceType.CPU] = self.cpu_cache_engine
        if cache_config.enable_ssd and cache_config.enable_p2p_ssd:
            # SSD blocks are published too: another node may read them straight out of this node's block files
            from .hie_cache_engine import HierarchyLRCacheEngine, get_node_registry
            self.node_registry = self.node_registry or get_node_registry(cache_config, model_config)
            self.ssd_cache_engine = HierarchyLRCacheEngine(DeviceType.SSD, cache_config.num_ssd_blocks,
                                                           registry=self.node_registry, **common)
            self.cache_engines[DeviceType.SSD] = self.ssd_cache_engine
        elif cache_config.enable_ssd:
            self.ssd_cache_engine = CacheEngine(DeviceType.SSD, cache_config.num_ssd_blocks, **common)
            self.cache_engines[DeviceType.SSD] = self.ssd_cache_engine
        if cache_config.enable_remote and cache_config.num_remote_blocks and \
                not cache_config.use_mooncake_store_backend:
            if cache_config.enable_3rd_remote:
                # a remote file system every node mounts: each node writes files of its own, publishes which
                # blocks they hold, and reads the other nodes' files (the role PCFS has in the reference:
                # flexkv/cache/hie_cache_engine.py:561-643, flexkv/cache/cache_engine.py:1024-1033)
                from .hie_cache_engine import HierarchyLRCacheEngine, get_node_registry
                self.node_registry = self.node_registry or get_node_registry(cache_config, model_config)
                self.remote_cache_engine = HierarchyLRCacheEngine(DeviceType.REMOTE, cache_config.num_remote_blocks,
                                                                  registry=self.node_registry, **common)
            else:
                self.remote_cache_engine = CacheEngine(DeviceType.REMOTE, cache_config.num_remote_blocks, **common)
            self.cache_engines[DeviceType.REMOTE] = self.remote_cache_engine
        if not self.cache_engines:
            raise ValueError("at least one cache tier must be enabled")
        if self.cpu_cache_engine is None:
            raise ValueError("the host tier is the staging area of every other tier and must be enabled")
        self.remote_backend = None          # key-addressed store; None = block-addressed index or no remote tier
        # engines without a prefetch hook may let compute-path gets read the key-addressed store in the graph
        self._store_in_graph = os.environ.get("FLEXKV_REMOTE_STORE_IN_GRAPH", "0") == "1"
        if cache_config.enable_remote and cache_config.use_mooncake_store_backend:
            from ..external.remote_store import get_backend
            self.set_remote_backend(get_backend(cache_config))
        self.peer_directory = None
        if cache_config.enable_p2p_gpu:
            from ..parallel.peer_directory import GpuPeerDirectory
            self.peer_directory = GpuPeerDirectory()
        # sliding-window snapshots ride on the host tier's nodes
        self.swa_ops = None
        swa_cfg = cache_config.swa.for_cache_tier(DeviceType.CPU) if cache_config.swa is not None else None
        if swa_cfg is not None and self.cpu_cache_engine is not None:
            from ..swa import SWAHostPool
            from .swa_cache_engine import SWAOpConstructor
            self.cpu_cache_engine.attach_swa(SWAHostPool(swa_cfg))
            self.swa_ops = SWAOpConstructor(self)
            # deeper window tiers: snapshots are written through beside the tier's blocks
            for dev, eng in ((DeviceType.SSD, self.ssd_cache_engine), (DeviceType.REMOTE, self.remote_cache_engine)):
                tier_cfg = cache_config.swa.for_cache_tier(dev)
                if tier_cfg is not None and eng is not None:
                    eng.attach_swa(SWAHostPool(tier_cfg))
        self._metrics = None
        self._evict_log = EvictionLogAggregator()
        for eng in self.cache_engines.values():
            eng.on_evict.append(self._on_evict)
        # warm restart: mount the SSD index that the last clean shutdown left beside the files
        self.ssd_blocks_restored = 0
        if self.ssd_cache_engine is not None and persist.persist_enabled(cache_config):
            self.ssd_blocks_restored = persist.load_index(cache_config, model_config, self.ssd_cache_engine)
        self.event_listeners: List[Any] = []   # objects with publish_stored / publish_removed

    # ---- observers ------------------------------------------------------------
    def set_metrics_collector(self, collector) -> None:
        self._metrics = collector
        self._update_mempool_metrics()

    checkpoint_valid = False     # an index image written while running is still true to the SSD files

    def checkpoint_ssd_index(self) -> bool:
        """Writes the SSD index now. The image stays valid only until the tier frees a block (which it is
        about to overwrite): the first SSD eviction after the call removes the image again, so a restart never
        mounts an index that names rewritten blocks."""
        if self.ssd_cache_engine is None or not persist.persist_enabled(self.cache_config):
            return False
        with self._cache_tree_lock:
            ok = persist.save_index(self.cache_config, self.model_config, self.ssd_cache_engine) is not None
            self.checkpoint_valid = ok
        return ok

    def _on_evict(self, device: DeviceType, blocks: np.ndarray, hashes: np.ndarray) -> None:
        if device == DeviceType.SSD and self.checkpoint_valid:
            self.checkpoint_valid = False
            persist.discard_index(self.cache_config)
        self._evict_log.record(device.name, len(blocks))
        if self._metrics is not None:
            self._metrics.record_eviction(device.name, len(blocks))
        for l in self.event_listeners:
            l.publish_removed(device, hashes)

    def _update_mempool_metrics(self) -> None:
        if self._metrics is None:
            return
        for d, e in self.cache_engines.items():
            self._metrics.set_mempool(d.name, e.num_total_blocks, e.mempool.num_free_blocks)

    # ---- public planner entry points -----------------------------------------------
    def reset(self) -> None:
        with self._cache_tree_lock:
            for e in self.cache_engines.values():
                e.reset()
            self._update_mempool_metrics()

    def shutdown(self) -> None:
        """Saves the SSD index when the tier persists (the data plane has stopped by now, so every
        ready block is on disk) and leaves the cross-node registry (withdraws published blocks,
        stops the heartbeat)."""
        if self.ssd_cache_engine is not None and persist.persist_enabled(self.cache_config) and \
                not self._index_saved:
            self._index_saved = True
            with self._cache_tree_lock:
                persist.save_index(self.cache_config, self.model_config, self.ssd_cache_engine)
        for e in self.cache_engines.values():
            if hasattr(e, "shutdown"):
                e.shutdown()
        if self.node_registry is not None:
            self.node_registry.stop(unregister=True)
            self.node_registry = None

    def _prepare(self, token_ids: np.ndarray, token_mask: Optional[np.ndarray], slot_mapping: Optional[np.ndarray]
                 ) -> Tuple[np.ndarray, np.ndarray, int, int, int]:
        """Validated inputs plus the block range ``[bstart, bend)`` the mask selects. Without a mask (the usual
        call) the range is the whole aligned prefix and nothing is scanned."""
        if token_ids.ndim != 1:
            raise ValueError("token_ids must be 1-D")
        token_ids = np.ascontiguousarray(token_ids, dtype=np.int64)
        n = token_ids.shape[0]
        tpb = self.tokens_per_block
        aligned = (n // tpb) * tpb
        if slot_mapping is not None and slot_mapping.ndim != 1:
            raise ValueError("slot_mapping must be 1-D")
        if token_mask is None:
            if slot_mapping is not None and slot_mapping.size != n:
                raise ValueError(f"slot_mapping has {slot_mapping.size} entries, token_mask selects {n} tokens")
            token_mask = np.ones(n, dtype=np.bool_)
            token_mask[aligned:] = False
            return token_ids, token_mask, aligned, 0, aligned // tpb
        token_mask = np.array(token_mask, dtype=np.bool_, copy=True)
        if token_mask.shape != token_ids.shape:
            raise ValueError(f"token_mask has {token_mask.size} entries for {token_ids.size} tokens")
        if slot_mapping is not None:
            selected = int(token_mask.sum())
            if slot_mapping.size != selected:
                raise ValueError(f"slot_mapping has {slot_mapping.size} entries, token_mask selects "
                                 f"{selected} tokens")
        token_mask[aligned:] = False
        bstart, bend = _block_range(token_mask, tpb)
        return token_ids, token_mask, aligned, bstart, bend

    def _empty(self, token_mask: np.ndarray):
        handle = TransferPlanHandle(lambda: None, lambda: None)
        return TransferOpGraph.create_empty_graph(), np.zeros_like(token_mask, dtype=np.bool_), handle, {}, -1

    def _finish(self, plan: TransferPlan, is_put: bool):
        graph = plan.graph
        if len(plan.finished_ops_ids) == 1:
            end_op = plan.finished_ops_ids[0]
        elif plan.finished_ops_ids:
            end_op = graph.add_virtual_op(plan.finished_ops_ids)
        else:
            end_op = -1
        for dev, lst in plan.nodes.items():
            for node, _ in lst:
                self.cache_engines[dev].lock_node(node)
        handle = TransferPlanHandle(complete=lambda: self._complete_plan(plan, is_put),
                                    abort=lambda: self._abort_plan(plan))
        handle.plan = plan        # the task layer reads plan.partial_blocks of a prefetch
        self._update_mempool_metrics()
        return graph, handle, plan.op_callback_dict, end_op

    def get(self, request_id: int, token_ids: np.ndarray, token_mask: Optional[np.ndarray],
            slot_mapping: Optional[np.ndarray], dp_client_id: int = 0, namespace: Optional[List[str]] = None,
            cpu_only: bool = False, prefetch: bool = False, swa_aware: bool = False):
        """Returns ``(graph, return_mask, plan_handle, op_callbacks, task_end_op_id)``."""
        token_ids, token_mask, aligned, bstart, bend = self._prepare(token_ids, token_mask, slot_mapping)
        if aligned == 0 or bend <= bstart:
            return self._empty(token_mask)
        tpb = self.tokens_per_block
        gpu_blocks = None
        if slot_mapping is not None:
            gpu_blocks = slot_mapping_to_block_ids(slot_mapping, tpb)[:bend - bstart]
        seq = SequenceMeta(token_ids[:aligned], tpb, namespace)
        with self._cache_tree_lock:
            swa_src = None
            if swa_aware and self.swa_ops is not None and self.swa_ops.enabled and not prefetch:
                # joint gate: only a prefix that ends where a window snapshot sits can be resumed
                m = self.cpu_cache_engine.match(seq)
                swa_src = (self.cpu_cache_engine, m.last_swa_node, int(m.swa_slot), int(m.swa_hit_blocks))
                for tier in (self.ssd_cache_engine, self.remote_cache_engine):
                    if tier is not None and tier.swa_enabled and not cpu_only:
                        mt = tier.match(seq)
                        if int(mt.swa_hit_blocks) > swa_src[3]:      # a deeper snapshot sits on this tier
                            swa_src = (tier, mt.last_swa_node, int(mt.swa_slot), int(mt.swa_hit_blocks))
                bend = min(bend, swa_src[3])
                if bend <= bstart:
                    return self._empty(token_mask)
                if swa_src[0] is self.cpu_cache_engine:
                    cpu_only = True                 # the host snapshot needs no deeper tier
                if gpu_blocks is not None:
                    gpu_blocks = gpu_blocks[:bend - bstart]
            plan = self._get_impl_local(seq, bstart, bend, gpu_blocks, dp_client_id, cpu_only, prefetch)
            if plan is None:
                return self._empty(token_mask)
            if swa_src is not None:
                if plan.num_gpu_blocks_to_transfer < bend - bstart:
                    # the full-KV plan fell short of the snapshot's position: the snapshot is useless
                    self._discard_plan(plan)
                    return self._empty(token_mask)
                src_eng, src_node, src_slot, _ = swa_src
                host_slot, stage_in = src_slot, None
                if src_eng is not self.cpu_cache_engine:
                    # SSD / remote snapshot: staged through a host slot that the plan gives back at its end
                    host_slot = self.cpu_cache_engine.alloc_swa_slot()
                    if host_slot is None:
                        self._discard_plan(plan)
                        return self._empty(token_mask)
                    hop = TransferType.DISK2H if src_eng is self.ssd_cache_engine else TransferType.REMOTE2H
                    stage_in = self.swa_ops.build_swa_op(plan.graph, hop, [src_slot], [host_slot], dp_client_id)
                    plan.swa_pending[stage_in.op_id] = host_slot
                op = self.swa_ops.build_get_chain(plan.graph, host_slot, dp_client_id)
                if op is not None:
                    if stage_in is not None:
                        plan.graph.add_dependency(op.op_id, stage_in.op_id)
                    src_eng.index.lock_swa(src_node)
                    plan.swa_locked.append((src_eng, src_node))
                    plan.finished_ops_ids = list(plan.finished_ops_ids) + [op.op_id]
            graph, handle, cbs, end_op = self._finish(plan, is_put=False)
        mask = np.zeros_like(token_mask, dtype=np.bool_)
        mask[bstart * tpb:(bstart + plan.num_gpu_blocks_to_transfer) * tpb] = True
        return graph, mask, handle, cbs, end_op

    def put(self, request_id: int, token_ids: np.ndarray, token_mask: Optional[np.ndarray],
            slot_mapping: Optional[np.ndarray], dp_client_id: int = 0, namespace: Optional[List[str]] = None):
        token_ids, token_mask, aligned, bstart, bend = self._prepare(token_ids, token_mask, slot_mapping)
        if aligned == 0 or bend <= bstart:
            return self._empty(token_mask)
        tpb = self.tokens_per_block
        if bstart != 0:
            raise ValueError("put: token_mask must select a prefix of the sequence")
        gpu_blocks = None
        if slot_mapping is not None:
            gpu_blocks = slot_mapping_to_block_ids(slot_mapping, tpb)[:bend]
        seq = SequenceMeta(token_ids[:aligned], tpb, namespace)
        with self._cache_tree_lock:
            plan = self._put_impl_local(seq, bend, gpu_blocks, dp_client_id)
            if plan is None:
                return self._empty(token_mask)
            graph, handle, cbs, end_op = self._finish(plan, is_put=True)
        mask = np.zeros_like(token_mask, dtype=np.bool_)
        lo = plan.skipped_gpu_blocks * tpb
        mask[lo:lo + plan.num_gpu_blocks_to_transfer * tpb] = True
        return graph, mask, handle, cbs, end_op

    # ---- GET ------------------------------------------------------------------------
    def _get_impl_local(self, seq: SequenceMeta, bstart: int, bend: int, gpu_blocks: Optional[np.ndarray],
                        dp_client_id: int, cpu_only: bool, prefetch: bool) -> Optional[TransferPlan]:
        cpu, ssd = self.cpu_cache_engine, (None if cpu_only else self.ssd_cache_engine)
        cpu_m = cpu.match(seq)
        ssd_m = ssd.match(seq) if ssd is not None else None
        cpu_hit = min(cpu_m.num_ready_matched_blocks, bend)
        ssd_hit = min(ssd_m.num_ready_matched_blocks, bend) if ssd_m is not None else 0
        if ssd_hit <= cpu_hit:
            ssd_m, ssd_hit = None, 0
        if self._metrics is not None:
            self._metrics.record_match("CPU", cpu_hit, bend - cpu_hit)
            if ssd is not None:
                self._metrics.record_match("SSD", ssd_hit, bend - ssd_hit)
        # Blocks that another rank holds in HBM come over NVLink instead of PCIe:
        # fragment 0 = [bstart, p_end) from peers, then host and SSD cover the rest.
        f0, peer_ranks, peer_blocks = 0, None, None
        if self.peer_directory is not None and not prefetch:
            f0, peer_ranks, peer_blocks = self.peer_directory.match_prefix(seq.block_hashes[:bend], dp_client_id,
                                                                           start=bstart, lease=True)
        p_end = bstart + f0
        end = max(cpu_hit, ssd_hit, p_end)
        lo1 = max(bstart, p_end)
        f1 = max(0, cpu_hit - lo1)                        # blocks [lo1, cpu_hit) from the host pool
        f2_lo = max(lo1, cpu_hit)
        f2 = max(0, max(cpu_hit, ssd_hit) - f2_lo)        # blocks [f2_lo, ...) from SSD
        if prefetch:
            f1 = 0
        # fragment 3: blocks only the remote tier has, beyond everything local
        f3, f3_lo, remote_m = 0, 0, None
        use_gds_early = bool(self.cache_config.enable_gds) and not prefetch
        # A key-addressed store sits behind a network: a get on the compute path stays on the local tiers and a
        # miss is recomputed; only a prefetch pulls from the store, ahead of scheduling
        # (reference: flexkv/cache/cache_engine.py:885-899 resolve_get_cache_strategy).
        store_in_graph = self.remote_backend is None or prefetch or self._store_in_graph
        if (self.remote_backend is not None or self.remote_cache_engine is not None) and not cpu_only \
                and not use_gds_early and store_in_graph:
            r_hit, remote_m = self._remote_hit(seq, bend)
            f3_lo = max(bstart, end)
            f3 = max(0, r_hit - f3_lo)
        # fragment 3 may instead come from another node's host pool when that node holds a longer prefix
        peer_host_nids, peer_is_ssd, peer_is_remote = None, False, False
        if self.node_registry is not None and not cpu_only and not use_gds_early and hasattr(cpu, "match_remote"):
            pm = cpu.match_remote(seq, bend)
            if pm.num_matched_blocks > max(end, f3_lo + f3):
                f3_lo = max(bstart, end)
                f3 = pm.num_matched_blocks - f3_lo
                peer_host_nids = pm.node_ids[f3_lo:f3_lo + f3]
                peer_host_src = pm.physical_blocks[f3_lo:f3_lo + f3]
                remote_m = None
        # ... or from another node's SSD tier when that reaches further still (read out of its block files)
        if self.node_registry is not None and not cpu_only and not use_gds_early and \
                hasattr(self.ssd_cache_engine, "match_remote"):
            sm = self.ssd_cache_engine.match_remote(seq, bend)
            if sm.num_matched_blocks > max(end, f3_lo + f3):
                f3_lo = max(bstart, end)
                f3 = sm.num_matched_blocks - f3_lo
                peer_host_nids = sm.node_ids[f3_lo:f3_lo + f3]
                peer_host_src = sm.physical_blocks[f3_lo:f3_lo + f3]
                peer_is_ssd, remote_m = True, None
        # ... or out of the files another node wrote to the remote file system all nodes mount
        if self.node_registry is not None and not cpu_only and not use_gds_early and \
                hasattr(self.remote_cache_engine, "match_remote"):
            rm = self.remote_cache_engine.match_remote(seq, bend)
            if rm.num_matched_blocks > max(end, f3_lo + f3):
                f3_lo = max(bstart, end)
                f3 = rm.num_matched_blocks - f3_lo
                peer_host_nids = rm.node_ids[f3_lo:f3_lo + f3]
                peer_host_src = rm.physical_blocks[f3_lo:f3_lo + f3]
                peer_is_ssd, peer_is_remote, remote_m = False, True, None
        if f0 + f1 + f2 + f3 == 0:
            return None
        graph = TransferOpGraph()
        plan = TransferPlan(graph)
        cpu_phys = cpu_m.physical_blocks
        use_gds = bool(self.cache_config.enable_gds) and not prefetch
        staging = _EMPTY
        stage_node = None
        if f2 > 0 and not use_gds:
            staging = cpu.take(f2, protected_node=cpu_m.last_node, strict=False)
            if len(staging) < f2:
                cpu.recycle(staging)
                if self._metrics is not None:
                    self._metrics.record_allocation_failure("CPU")
                if f0 + f1 == 0:
                    return None
                f2, staging = 0, _EMPTY
        ops_done: List[int] = []
        disk_op = None
        if f0 > 0:
            peer_op = TransferOp(graph.graph_id, TransferType.PEERD2D, peer_blocks,
                                 gpu_blocks[:f0] if gpu_blocks is not None else _EMPTY, dp_client_id=dp_client_id,
                                 gpu_side=None if gpu_blocks is not None else "dst", gpu_bind="head",
                                 remote_node_ids=peer_ranks)
            graph.add_transfer_op(peer_op)
            ops_done.append(peer_op.op_id)
            plan.peer_leases = (peer_ranks, peer_blocks)
        if f2 > 0:
            ssd_src = ssd_m.physical_blocks[f2_lo:f2_lo + f2]
            if use_gds:
                disk_op = TransferOp(graph.graph_id, TransferType.DISK2D, ssd_src,
                                     gpu_blocks[f0 + f1:f0 + f1 + f2] if gpu_blocks is not None else _EMPTY,
                                     dp_client_id=dp_client_id,
                                     gpu_side=None if gpu_blocks is not None else "dst", gpu_bind="tail")
            else:
                disk_op = TransferOp(graph.graph_id, TransferType.DISK2H, ssd_src, staging, dp_client_id=dp_client_id)
            graph.add_transfer_op(disk_op)
            plan.nodes.setdefault(DeviceType.SSD, []).append((ssd_m.last_ready_node, 0))
            if not use_gds:
                # keep the staged copy as cache content when it extends a fully ready host prefix
                contiguous = cpu_m.num_matched_blocks == cpu_m.num_ready_matched_blocks == f2_lo
                if contiguous:
                    try:
                        stage_node = cpu.insert(seq, staging, num_insert_blocks=f2_lo + f2, is_ready=False,
                                                match_result=cpu_m)
                    except RuntimeError:
                        stage_node = None
                if stage_node is not None:
                    plan.nodes.setdefault(DeviceType.CPU, []).append((stage_node, 0))
                    plan.inserted.setdefault(DeviceType.CPU, []).append(stage_node)
                    node, n = stage_node, f2
                    plan.op_callback_dict[disk_op.op_id] = lambda node=node, n=n: cpu.set_ready(node, True, n)
                else:
                    plan.buffer_to_free[DeviceType.CPU] = staging
        remote_op, staging3 = None, _EMPTY
        if f3 > 0:
            staging3 = cpu.take(f3, protected_node=cpu_m.last_node, strict=False)
            if len(staging3) < f3:
                cpu.recycle(staging3)
                f3, staging3 = 0, _EMPTY
        if f3 > 0:
            hashes3 = seq.block_hashes[f3_lo:f3_lo + f3]
            src3 = remote_m.physical_blocks[f3_lo:f3_lo + f3] if remote_m is not None else np.zeros(f3, dtype=np.int64)
            if peer_host_nids is not None:
                remote_op = TransferOp(graph.graph_id,
                                       TransferType.REMOTE2H if peer_is_remote else
                                       TransferType.PEERSSD2H if peer_is_ssd else TransferType.PEERH2H,
                                       peer_host_src, staging3,
                                       dp_client_id=dp_client_id, block_hashes=hashes3,
                                       remote_node_ids=peer_host_nids)
            else:
                remote_op = TransferOp(graph.graph_id, TransferType.REMOTE2H, src3, staging3,
                                       dp_client_id=dp_client_id, block_hashes=hashes3)
            graph.add_transfer_op(remote_op)
            if remote_m is not None:
                plan.nodes.setdefault(DeviceType.REMOTE, []).append((remote_m.last_ready_node, 0))
            # the pulled blocks become host cache content when they extend what the host tier holds contiguously
            node3 = None
            tail_ok = (stage_node is not None and f2_lo + f2 == f3_lo) or \
                (f2 == 0 and cpu_m.num_matched_blocks == cpu_m.num_ready_matched_blocks == f3_lo)
            if tail_ok:
                try:
                    node3 = cpu.insert(seq, staging3, num_insert_blocks=f3_lo + f3, is_ready=False,
                                       match_result=None if stage_node is not None else cpu_m)
                except (RuntimeError, ValueError):
                    node3 = None
            if node3 is not None and prefetch and remote_op.transfer_type == TransferType.REMOTE2H:
                # a prefetch may succeed for a prefix only: the staged node is replaced by one that holds the
                # blocks that arrived, the rest goes back to the pool, and the response mask shrinks
                remote_op.allow_partial = True
                plan.inserted.setdefault(DeviceType.CPU, []).append(node3)

                def _adopt(c, node=node3, lo=f3_lo, n=f3):
                    res = getattr(c, "block_results", None)
                    k = n if res is None else next((i for i, ok in enumerate(res) if not ok), n)
                    if k < n:
                        tail = cpu.index.truncate_unready_leaf(node, k)
                        cpu.recycle(tail)
                        plan.partial_blocks = (lo - bstart) + k
                    if k > 0:
                        cpu.set_ready(node, True, k)
                _adopt.wants_result = True
                plan.op_callback_dict[remote_op.op_id] = _adopt
            elif node3 is not None:
                plan.nodes.setdefault(DeviceType.CPU, []).append((node3, 0))
                plan.inserted.setdefault(DeviceType.CPU, []).append(node3)
                plan.op_callback_dict[remote_op.op_id] = lambda node=node3, n=f3: cpu.set_ready(node, True, n)
            else:
                prev = plan.buffer_to_free.get(DeviceType.CPU, _EMPTY)
                plan.buffer_to_free[DeviceType.CPU] = np.concatenate([prev, staging3])
        if prefetch:
            done = [o.op_id for o in (disk_op, remote_op) if o is not None]
            if not done:
                return None
            plan.finished_ops_ids = done
            plan.num_gpu_blocks_to_transfer = f2 + f3
            return plan
        h2d_src = np.concatenate([cpu_phys[lo1:lo1 + f1], staging, staging3]) if not use_gds \
            else cpu_phys[lo1:lo1 + f1]
        n_h2d = int(h2d_src.size)
        if n_h2d > 0:
            h2d = TransferOp(graph.graph_id, TransferType.H2D, h2d_src,
                             gpu_blocks[f0:f0 + n_h2d] if gpu_blocks is not None else _EMPTY,
                             dp_client_id=dp_client_id, gpu_side=None if gpu_blocks is not None else "dst",
                             gpu_bind="head", gpu_offset=f0)
            graph.add_transfer_op(h2d)
            if disk_op is not None and not use_gds:
                graph.add_dependency(h2d.op_id, disk_op.op_id)
            if remote_op is not None:
                graph.add_dependency(h2d.op_id, remote_op.op_id)
            ops_done.append(h2d.op_id)
            if f1 > 0:
                plan.nodes.setdefault(DeviceType.CPU, []).append((cpu_m.last_ready_node, 0))
        if disk_op is not None and use_gds:
            ops_done.append(disk_op.op_id)
        plan.finished_ops_ids = ops_done
        plan.num_gpu_blocks_to_transfer = f0 + f1 + f2 + f3
        return plan

    # ---- PUT ------------------------------------------------------------------------
    def _put_impl_local(self, seq: SequenceMeta, nb: int, gpu_blocks: Optional[np.ndarray], dp_client_id: int
                        ) -> Optional[TransferPlan]:
        cpu, ssd = self.cpu_cache_engine, self.ssd_cache_engine
        # matched (ready or still in flight) blocks are never offloaded twice
        cpu_m = cpu.match(seq)
        cpu_matched = min(cpu_m.num_matched_blocks, nb)
        need_cpu = nb - cpu_matched
        ssd_m, ssd_matched, need_ssd = None, 0, 0
        if ssd is not None:
            ssd_m = ssd.match(seq)
            ssd_matched = min(ssd_m.num_matched_blocks, nb)
            need_ssd = nb - ssd_matched
            # host blocks that another task is still filling cannot feed a disk write
            if need_ssd > 0 and nb - need_ssd < cpu_matched and cpu_m.num_ready_matched_blocks < cpu_matched:
                need_ssd = 0
        if need_cpu == 0 and need_ssd == 0:
            # Everything is on the local tiers already. If the remote tier misses part of it (an earlier upload
            # failed or was evicted there) and the host copy is complete and ready, the put becomes an upload
            # from the host blocks alone, without touching the GPU
            # (reference scenario: tests/test_mooncake_deferred_put.py:298-317).
            if cpu_m.num_ready_matched_blocks < nb or not self._remote_lacks(seq, nb):
                return None
        cpu_new = cpu.take(need_cpu, protected_node=cpu_m.last_node, strict=False) if need_cpu else _EMPTY
        if len(cpu_new) < need_cpu:
            cpu.recycle(cpu_new)
            if self._metrics is not None:
                self._metrics.record_allocation_failure("CPU")
            return None
        ssd_new = _EMPTY
        if need_ssd:
            ssd_new = ssd.take(need_ssd, protected_node=ssd_m.last_node, strict=False)
            if len(ssd_new) < need_ssd:
                ssd.recycle(ssd_new)
                cpu.recycle(cpu_new)
                if self._metrics is not None:
                    self._metrics.record_allocation_failure("SSD")
                return None
        graph = TransferOpGraph()
        plan = TransferPlan(graph)
        d2h = None
        if need_cpu:
            late = gpu_blocks is None
            d2h = TransferOp(graph.graph_id, TransferType.D2H,
                             _EMPTY if late else gpu_blocks[cpu_matched:nb], cpu_new, dp_client_id=dp_client_id,
                             gpu_side="src" if late else None, gpu_bind="head")
            graph.add_transfer_op(d2h)
            try:
                cpu_node = cpu.insert(seq, cpu_new, num_insert_blocks=nb, is_ready=False, match_result=cpu_m)
            except RuntimeError:
                cpu.recycle(cpu_new)
                ssd and ssd.recycle(ssd_new)
                raise
            plan.nodes.setdefault(DeviceType.CPU, []).append((cpu_node, 0))
            plan.inserted.setdefault(DeviceType.CPU, []).append(cpu_node)
            plan.op_callback_dict[d2h.op_id] = lambda node=cpu_node, n=need_cpu: cpu.set_ready(node, True, n)
        elif not cpu.index.is_root(cpu_m.last_node):
            plan.nodes.setdefault(DeviceType.CPU, []).append((cpu_m.last_node, 0))
        if need_ssd:
            cpu_all = np.concatenate([cpu_m.physical_blocks[:cpu_matched], cpu_new])
            disk = TransferOp(graph.graph_id, TransferType.H2DISK, cpu_all[nb - need_ssd:nb], ssd_new,
                              dp_client_id=dp_client_id)
            graph.add_transfer_op(disk)
            if d2h is not None:
                graph.add_dependency(disk.op_id, d2h.op_id)
            ssd_node = ssd.insert(seq, ssd_new, num_insert_blocks=nb, is_ready=False, match_result=ssd_m)
            plan.nodes.setdefault(DeviceType.SSD, []).append((ssd_node, 0))
            plan.inserted.setdefault(DeviceType.SSD, []).append(ssd_node)
            plan.op_callback_dict[disk.op_id] = lambda node=ssd_node, n=need_ssd: ssd.set_ready(node, True, n)
            if d2h is None:
                plan.finished_ops_ids = [disk.op_id]
        self._put_remote(seq, nb, cpu_m, cpu_matched, cpu_new, d2h, graph, plan, dp_client_id)
        if d2h is not None:
            plan.finished_ops_ids = [d2h.op_id]     # the caller may see success before the disk write ends
        if d2h is not None and self.swa_ops is not None and self.swa_ops.enabled:
            # snapshot of the window state after the last offloaded block, mounted on the new node
            slot = cpu.alloc_swa_slot()
            if slot is not None:
                chain = self.swa_ops.build_put_chain(graph, slot, dp_client_id)
                if chain.d2h_id is None:
                    cpu.swa_pool.free(slot)
                else:
                    swa_op = graph.get_op(chain.d2h_id)
                    plan.swa_pending[chain.d2h_id] = slot

                    # write-through to the deeper window tiers, onto the node this put created there
                    chained = []
                    for dev, hop in ((DeviceType.SSD, TransferType.H2DISK), (DeviceType.REMOTE, TransferType.H2REMOTE)):
                        tier = self.cache_engines.get(dev)
                        if tier is None or not tier.swa_enabled or not plan.inserted.get(dev):
                            continue
                        tier_slot = tier.alloc_swa_slot()
                        if tier_slot is None:
                            continue
                        tier_op = self.swa_ops.build_swa_op(graph, hop, [slot], [tier_slot], dp_client_id)
                        graph.add_dependency(tier_op.op_id, chain.d2h_id)
                        plan.swa_pending_tier[tier_op.op_id] = (tier, tier_slot)
                        chained.append((tier, tier_slot, tier_op, plan.inserted[dev][-1]))

                    def _mount(node=cpu_node, slot=slot, op=swa_op, oid=chain.d2h_id, chained=bool(chained)):
                        plan.swa_pending.pop(oid, None)
                        if op.transfer_type == TransferType.VIRTUAL or not cpu.index.alive(node):
                            cpu.swa_pool.free(slot)
                        elif cpu.mount_swa(node, slot) and chained:
                            # the slot feeds the tier writes: it must not be evicted and reused before they end
                            cpu.index.lock_swa(node)
                            plan.swa_locked.append((cpu, node))
                    plan.op_callback_dict[chain.d2h_id] = _mount
                    plan.finished_ops_ids = list(plan.finished_ops_ids) + [chain.d2h_id]
                    for tier, tier_slot, tier_op, tier_node in chained:
                        def _mount_tier(tier=tier, node=tier_node, s_=tier_slot, op=tier_op):
                            plan.swa_pending_tier.pop(op.op_id, None)
                            if op.transfer_type == TransferType.VIRTUAL or not tier.index.alive(node):
                                tier.swa_pool.free(s_)
                            else:
                                tier.mount_swa(node, s_)
                        plan.op_callback_dict[tier_op.op_id] = _mount_tier
        if graph.num_ops == 0:
            return None                                  # the remote tier could not take the upload either
        plan.skipped_gpu_blocks = cpu_matched
        plan.num_gpu_blocks_to_transfer = need_cpu
        return plan

    def _remote_lacks(self, seq: SequenceMeta, nb: int) -> bool:
        """True when a remote tier exists and holds fewer than the first `nb` blocks of the sequence."""
        if self.remote_backend is not None:
            return self.remote_backend.prefix_hit(seq.block_hashes[:nb]) < nb
        if self.remote_cache_engine is not None:
            return self.remote_cache_engine.match(seq, update_cache_info=False).num_matched_blocks < nb
        return False

    def _put_remote(self, seq, nb, cpu_m, cpu_matched, cpu_new, d2h, graph, plan, dp_client_id) -> None:
        """Write-through of the blocks the remote tier lacks (H2REMOTE after the GPU->host copy)."""
        if self.remote_backend is None and self.remote_cache_engine is None:
            return
        if cpu_m.num_ready_matched_blocks < cpu_matched:
            return                                   # host blocks of another in-flight put cannot be a source
        cpu_all = np.concatenate([cpu_m.physical_blocks[:cpu_matched], cpu_new])
        if self.remote_backend is not None:
            have = min(self.remote_backend.prefix_hit(seq.block_hashes[:nb]), nb)
            if have >= nb:
                return
            op = TransferOp(graph.graph_id, TransferType.H2REMOTE, cpu_all[have:nb],
                            np.zeros(nb - have, dtype=np.int64), dp_client_id=dp_client_id,
                            block_hashes=seq.block_hashes[have:nb])
        else:
            rem = self.remote_cache_engine
            rm = rem.match(seq)
            have = min(rm.num_matched_blocks, nb)
            if have >= nb:
                return
            new = rem.take(nb - have, protected_node=rm.last_node, strict=False)
            if len(new) < nb - have:
                rem.recycle(new)
                return
            op = TransferOp(graph.graph_id, TransferType.H2REMOTE, cpu_all[have:nb], new, dp_client_id=dp_client_id,
                            block_hashes=seq.block_hashes[have:nb])
            node = rem.insert(seq, new, num_insert_blocks=nb, is_ready=False, match_result=rm)
            plan.nodes.setdefault(DeviceType.REMOTE, []).append((node, 0))
            plan.inserted.setdefault(DeviceType.REMOTE, []).append(node)
            plan.op_callback_dict[op.op_id] = lambda node=node, n=nb - have: rem.set_ready(node, True, n)
        graph.add_transfer_op(op)
        if d2h is not None:
            graph.add_dependency(op.op_id, d2h.op_id)
        elif not plan.finished_ops_ids:
            plan.finished_ops_ids = [op.op_id]

    # ---- plan end --------------------------------------------------------------------
    def _complete_plan(self, plan: TransferPlan, is_put: bool) -> None:
        with self._cache_tree_lock:
            for dev, lst in plan.nodes.items():
                for node, _ in lst:
                    self.cache_engines[dev].unlock(node)
            for dev, ids in plan.buffer_to_free.items():
                self.cache_engines[dev].recycle(ids)
            self._release_peer(plan)
            self._release_swa(plan)
            # a node whose op callback never ran (op skipped) stays unready; drop it
            for dev, lst in plan.inserted.items():
                for node in lst:
                    eng = self.cache_engines[dev]
                    if eng.index.alive(node) and not eng.index.node_ready(node):
                        eng.rollback_unready_insert(node)
            self._update_mempool_metrics()

    def _abort_plan(self, plan: TransferPlan) -> None:
        with self._cache_tree_lock:
            for dev, lst in plan.nodes.items():
                for node, _ in lst:
                    self.cache_engines[dev].unlock(node)
            for dev, lst in plan.inserted.items():
                for node in lst:
                    self.cache_engines[dev].rollback_unready_insert(node)
            for dev, ids in plan.buffer_to_free.items():
                self.cache_engines[dev].recycle(ids)
            self._release_peer(plan)
            self._release_swa(plan)
            self._update_mempool_metrics()

    def _discard_plan(self, plan: TransferPlan) -> None:
        """Gives back what a plan reserved before its nodes were locked (it never launches)."""
        for dev, lst in plan.inserted.items():
            for node in lst:
                self.cache_engines[dev].rollback_unready_insert(node)
        for dev, ids in plan.buffer_to_free.items():
            self.cache_engines[dev].recycle(ids)
        self._release_peer(plan)

    def _release_swa(self, plan: TransferPlan) -> None:
        cpu = self.cpu_cache_engine
        for eng, node in plan.swa_locked:
            if eng.index.alive(node):
                eng.index.unlock_swa(node)
        plan.swa_locked = []
        for slot in plan.swa_pending.values():      # side ops that never completed, staging slots of gets
            cpu.swa_pool.free(slot)
        plan.swa_pending = {}
        for tier, slot in plan.swa_pending_tier.values():
            tier.swa_pool.free(slot)
        plan.swa_pending_tier = {}

    def _release_peer(self, plan: TransferPlan) -> None:
        if plan.peer_leases is not None and self.peer_directory is not None:
            self.peer_directory.release(*plan.peer_leases)
            plan.peer_leases = None

    def set_remote_backend(self, backend) -> None:
        """Key-addressed remote stores are probed by content key instead of a local index."""
        self.remote_backend = backend if backend is not None and backend.key_addressed else None

    def _remote_hit(self, seq: SequenceMeta, bend: int):
        """(blocks available remotely from block 0, remote block ids or None for key-addressed)."""
        if self.remote_backend is not None:
            return min(self.remote_backend.prefix_hit(seq.block_hashes[:bend]), bend), None
        if self.remote_cache_engine is not None:
            m = self.remote_cache_engine.match(seq)
            return min(m.num_ready_matched_blocks, bend), m
        return 0, None

    def publish_gpu_blocks(self, rank: int, token_ids: np.ndarray, gpu_block_ids: np.ndarray,
                           namespace: Optional[List[str]] = None) -> int:
        """Announces that `rank`'s GPU blocks hold the leading blocks of this sequence."""
        if self.peer_directory is None:
            return 0
        seq = SequenceMeta(np.ascontiguousarray(token_ids, dtype=np.int64), self.tokens_per_block, namespace)
        n = min(seq.num_blocks, len(gpu_block_ids))
        self.peer_directory.publish(rank, seq.block_hashes[:n], np.asarray(gpu_block_ids[:n], dtype=np.int64))
        return n

    def withdraw_gpu_blocks(self, rank: int, gpu_block_ids: np.ndarray) -> List[int]:
        if self.peer_directory is None:
            return []
        return self.peer_directory.withdraw_blocks(rank, np.asarray(gpu_block_ids, dtype=np.int64))

    def run_op_callback(self, cb: Callable, completed: Any = None) -> None:
        """Callbacks marked ``wants_result`` receive the completed op (per-block results)."""
        with self._cache_tree_lock:
            if getattr(cb, "wants_result", False):
                cb(completed)
            else:
                cb()
