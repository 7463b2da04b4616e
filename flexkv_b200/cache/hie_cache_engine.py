"""Host-tier cache engine that also knows what other nodes hold.

``HierarchyLRCacheEngine`` pairs a lease-aware local index (native ``LocalRadixTree``:
the tier's own radix index whose ready blocks are published with a lease) with a
read-only view of every other node (native ``DistributedRadixTree``). ``match_all``
returns both matches; the planner reads from a peer only where the peer's prefix is
longer than everything this node holds (reference: flexkv/cache/hie_cache_engine.py:
239-334 ``match_all``, :177-223 reset barrier; native halves csrc/dist/*).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .. import _native
from ..common.block import SequenceMeta
from ..common.config import GLOBAL_CONFIG_FROM_ENV
from ..common.debug import flexkv_logger
from ..common.transfer import DeviceType
from .cache_engine import CacheEngine
from .mempool import Mempool
from .registry import NodeRegistry, RegistryClient, RegistryMetaChannel, connect


@dataclass
class RemoteMatch:
    num_matched_blocks: int
    physical_blocks: np.ndarray     # int64, block ids in the owner's host pool
    node_ids: np.ndarray            # uint32, owner of every block


class HierarchyLRCacheEngine(CacheEngine):
    def __init__(self, device_type: DeviceType, num_total_blocks: int, tokens_per_block: int, *,
                 registry: NodeRegistry, channel=None, evict_ratio: float = 0.0, hit_reward_seconds: float = 0.0,
                 eviction_policy: str = "lru", slru_threshold: int = 2, evict_start_threshold: float = 1.0,
                 lease_ttl_ms: Optional[int] = None, renew_lease_ms: Optional[int] = None,
                 refresh_interval_ms: Optional[int] = None, safety_ttl_ms: Optional[int] = None,
                 start_threads: bool = True) -> None:
        env = GLOBAL_CONFIG_FROM_ENV
        # CacheEngine.__init__ would build a plain index; set the same fields by hand
        if num_total_blocks <= 0:
            raise ValueError(f"invalid num_total_blocks: {num_total_blocks}")
        self.device_type = device_type
        self.num_total_blocks = int(num_total_blocks)
        self.tokens_per_block = tokens_per_block
        self.evict_ratio = evict_ratio
        self.evict_start_threshold = evict_start_threshold
        self.accel = True
        self.registry = registry
        if registry.node_id is None:
            registry.register()
        self.node_id = int(registry.node_id)
        # record families of the three published tiers (the reference names its shared remote tier after PCFS)
        kind = {DeviceType.CPU: "CPUB", DeviceType.SSD: "SSDB", DeviceType.REMOTE: "PCFSB"}.get(device_type, "CPUB")
        if channel is None:
            # a registry in a Redis server gets the native channel, the in-box registry the Python one
            native = getattr(registry.client, "native_channel", None)
            channel = native(kind) if callable(native) else RegistryMetaChannel(registry.client, kind)
        self.channel = channel
        lease = int(lease_ttl_ms if lease_ttl_ms is not None else env.lease_ttl_ms)
        renew = int(renew_lease_ms if renew_lease_ms is not None else env.renew_lease_ms)
        refresh = int(refresh_interval_ms if refresh_interval_ms is not None else 100)
        # how often the read-only view of the other nodes' blocks is rebuilt (FLEXKV_REBUILD_INTERVAL_MS)
        rebuild = int(refresh_interval_ms if refresh_interval_ms is not None else getattr(env, "rebuild_interval_ms", 2000))
        safety = int(safety_ttl_ms if safety_ttl_ms is not None else getattr(env, "safety_ttl_ms", 100))
        self.index = _native.C.LocalRadixTree(self.node_id, tokens_per_block, self.num_total_blocks, eviction_policy,
                                              float(hit_reward_seconds), self.channel, lease_ttl_ms=lease,
                                              renew_margin_ms=min(renew, max(1, lease - 1)),
                                              refresh_interval_ms=refresh, safety_ttl_ms=safety,
                                              start_thread=start_threads)
        self.remote_view = _native.C.DistributedRadixTree(self.node_id, self.channel, refresh_interval_ms=rebuild,
                                                          safety_ttl_ms=safety, start_thread=start_threads)
        self.mempool = Mempool(self.num_total_blocks, native=True)
        self.on_evict, self.on_insert = [], []
        self.num_evicted_total = 0
        self._reset_epoch = 0

    # ---- matching ---------------------------------------------------------------------
    def match_remote(self, seq: SequenceMeta, limit: Optional[int] = None) -> RemoteMatch:
        n = seq.num_blocks if limit is None else min(limit, seq.num_blocks)
        k, pbs, nids = self.remote_view.match_prefix(seq.block_hashes, n)
        return RemoteMatch(int(k), pbs, nids)

    def match_all(self, seq: SequenceMeta, update_cache_info: bool = True):
        """(local match, remote match, "local" | "remote") — remote wins only when longer."""
        local = self.match(seq, update_cache_info)
        remote = self.match_remote(seq)
        winner = "remote" if remote.num_matched_blocks > local.num_ready_matched_blocks else "local"
        return local, remote, winner

    def refresh(self) -> None:
        """One synchronous publish + view rebuild (tests and shutdown paths; the native
        threads do this periodically otherwise)."""
        self.index.refresh_once()
        self.remote_view.refresh_once()

    # ---- lifecycle ----------------------------------------------------------------------
    def reset(self, barrier_timeout: Optional[float] = None) -> None:
        """Drops every local block, withdraws the published records and waits until all
        live nodes acknowledged the same reset epoch (FLEXKV_RESET_BARRIER_TIMEOUT_MS / _POLL_MS)."""
        env = GLOBAL_CONFIG_FROM_ENV
        if barrier_timeout is None:
            barrier_timeout = float(getattr(env, "reset_barrier_timeout_ms", 60000)) / 1e3
        self.index.reset()
        self.mempool.reset()
        self._reset_epoch += 1
        if not self.registry.reset_barrier(self._reset_epoch, timeout=barrier_timeout,
                                           poll=float(getattr(env, "reset_barrier_poll_ms", 50)) / 1e3):
            flexkv_logger.warning("reset barrier %d timed out; some nodes may still list old blocks",
                                  self._reset_epoch)
        self.remote_view.refresh_once()

    def shutdown(self) -> None:
        self.index.shutdown()
        self.remote_view.shutdown()
        try:
            self.channel.clear_node(self.node_id)
        except Exception:  # noqa: BLE001
            pass


def get_node_registry(cache_config, model_config=None) -> NodeRegistry:
    """One registry membership per CacheConfig, shared by the planner (index publication)
    and the data plane (peer pool lookup). The address comes from the redis_host/redis_port
    fields; "inproc[:name]" keeps the store inside the process."""
    reg = getattr(cache_config, "_node_registry_obj", None)
    if reg is not None:
        return reg
    client: RegistryClient = connect(cache_config.redis_host, int(cache_config.redis_port),
                                     getattr(cache_config, "redis_password", None))
    pp_rank = getattr(model_config, "pp_rank", 0) if model_config is not None else 0
    pp_size = getattr(model_config, "pp_size", 1) if model_config is not None else 1
    reg = NodeRegistry(client, ip=cache_config.local_ip or "127.0.0.1", pp_rank=pp_rank, pp_size=pp_size,
                       node_ttl_seconds=float(cache_config.node_ttl_seconds or 30))
    reg.register()
    reg.start_heartbeat()
    object.__setattr__(cache_config, "_node_registry_obj", reg)
    return reg
