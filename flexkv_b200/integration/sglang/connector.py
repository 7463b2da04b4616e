"""SGLang HiCache-style connector.

Every rank owns a ``KVTPClient`` (registers its ``2L`` K/V buffers); only the sync
leader owns a ``KVManager``. Lookups, stores and loads are decided on the leader
and scattered to the other ranks as manifests so that all ranks act on the same
matched length (flexkv/integration/sglang/connector.py:116-2291, start-up
:190-333, lookup :460-586, retrieve :605-694, layerwise load :696-955, store
:1011-1182, prefetch :1281-1406, reset :1424).
"""
from __future__ import annotations

import atexit
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...common.config import GLOBAL_CONFIG_FROM_ENV
from ...common.request import KVResponseStatus
from ...common.storage import KVCacheLayout, KVCacheLayoutType
from ..config import FlexKVConfig
from ..stats import FlexKVStats
from .comm import FlexKVComm, FlexKVLayerDoneCounter
from .pools import (ResolvedPool, build_swa_slot_mapping, layer_group_specs, resolve_kv_pool,
                    window_pool_config)


@dataclass
class _PendingLoad:
    rid: str
    task_id: int
    matched_tokens: int
    start_block: int


def sglang_gpu_layout(k_buffers: Sequence[torch.Tensor], page_size: int, use_mla: bool) -> KVCacheLayout:
    t = k_buffers[0]
    L = len(k_buffers)
    tokens = t.shape[0]
    if use_mla:
        return KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, tokens // page_size, page_size, 1, t.shape[-1],
                             is_mla=True)
    return KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, tokens // page_size, page_size, t.shape[-2], t.shape[-1])


_UNSET = object()


def swa_transfer_enabled_from_env() -> bool:
    return bool(int(os.environ.get("FLEXKV_ENABLE_SWA_TRANSFER", "1")))


class FlexKVConnector:
    def __init__(self, flexkv_config: Optional[FlexKVConfig] = None, page_size: int = 0, tp_rank: int = 0,
                 tp_size: int = 1, pp_rank: int = 0, pp_size: int = 1, dp_rank: int = 0, cp_rank: int = 0,
                 cp_size: int = 1, comm: Optional[FlexKVComm] = None, kv_manager: Any = None, register: bool = True,
                 hand_off_slot_mapping: bool = False, *, sgl_model_config: Any = None, server_args: Any = None,
                 kvcache: Any = None, attn_cp_rank: Optional[int] = None, pp_group: Any = None,
                 attn_tp_group: Any = None, attn_cp_group: Any = None) -> None:
        """``hand_off_slot_mapping``: set on ONE rank of every node other than the leader's when the group
        spans nodes. That node's transfer manager receives the leader's graphs with the GPU side unbound; this
        rank sends it the pages its node allocated for each task (flexkv/integration/sglang/connector.py:2199-2204).

        The keyword-only arguments are the reference's constructor (``sgl_model_config``, ``server_args``,
        ``kvcache``, ``attn_cp_rank`` and the engine's process groups, as its SGLang patch passes them): the
        configuration is then read off the engine's objects, group sizes off the groups, the pool geometry off
        ``kvcache``, and the pool is registered at the end of construction."""
        pool = None
        if flexkv_config is None:
            if sgl_model_config is None:
                raise TypeError("FlexKVConnector needs a FlexKVConfig, or the engine's model config and server args")

            def size(g: Any) -> int:
                if g is None:
                    return 1
                n = getattr(g, "world_size", None)
                return int(n if n is not None else g.size())
            tp_size, cp_size, pp_size = size(attn_tp_group), size(attn_cp_group), size(pp_group)
            cp_rank = int(attn_cp_rank or 0)
            flexkv_config = FlexKVConfig.from_env()
            flexkv_config.post_init_from_sglang_config(server_args, sgl_model_config, int(page_size), tp_size=tp_size,
                                                       pp_size=pp_size, cp_size=cp_size,
                                                       dp_size=int(getattr(server_args, "dp_size", 1) or 1))
            if kvcache is not None:
                pool = FlexKVConnector.configure_for_pool(flexkv_config, kvcache, int(page_size))
        self.cfg = flexkv_config
        self.hand_off_slot_mapping = bool(hand_off_slot_mapping)
        self.any_hand_off: Optional[bool] = None      # agreed over the group at the first load or store
        self.T = page_size
        self.tp_rank, self.tp_size, self.pp_rank, self.dp_rank = tp_rank, tp_size, pp_rank, dp_rank
        self.comm = comm or FlexKVComm(tp_size=tp_size, cp_size=cp_size, pp_size=pp_size)
        self.is_leader = self.comm.is_leader
        self.stats = FlexKVStats()
        self.layerwise = bool(GLOBAL_CONFIG_FROM_ENV.enable_layerwise_transfer)
        self.layer_counter: Optional[FlexKVLayerDoneCounter] = None
        self.mgr = kv_manager
        if self.is_leader and self.mgr is None:
            from ...kvmanager import KVManager
            self.mgr = KVManager(flexkv_config.model_config, flexkv_config.cache_config, dp_client_id=dp_rank,
                                 server_recv_port=flexkv_config.server_recv_port,
                                 gpu_register_port=flexkv_config.gpu_register_port)
            self.mgr.start()
        self._pending_loads: Dict[str, _PendingLoad] = {}
        self._stores: Dict[str, int] = {}
        self._prefetch: Dict[str, int] = {}
        self._launched_loads: List[int] = []      # loads started through the single-request layerwise form
        # prefetching pays only where a tier below the host pool exists (flexkv/integration/sglang/connector.py:302-306);
        # a key-addressed remote store is read by prefetches alone, so it must be on with one
        cc = flexkv_config.cache_config
        self.prefetch_enabled = bool(cc.enable_ssd or cc.enable_remote or cc.enable_kv_sharing)
        from ...common.config import assert_mooncake_prefetch_ready
        assert_mooncake_prefetch_ready(cc, self.prefetch_enabled)
        self._client = None
        if register:
            from ...server.client import KVTPClient
            dev = torch.cuda.current_device() if torch.cuda.is_available() else 0
            self._client = KVTPClient(flexkv_config.gpu_register_port, dp_rank, dev, tp_rank=cp_rank * tp_size + tp_rank,
                                      pp_rank=pp_rank)
        atexit.register(self.shutdown)
        if kvcache is not None and sgl_model_config is not None and self._client is not None:
            self.register_kv_pool(kvcache, pool)

    # ---- start-up ---------------------------------------------------------------------
    def register_kv_buffers(self, k_buffers: Sequence[torch.Tensor], v_buffers: Optional[Sequence[torch.Tensor]] = None,
                            group_id: int = -1) -> None:
        use_mla = v_buffers is None or self.cfg.model_config.use_mla
        layout = sglang_gpu_layout(k_buffers, self.T, use_mla)
        # every rank must agree on the number of pages it can address
        nb = self.comm.all_reduce_min(layout.num_block)
        layout = layout._replace(num_block=nb)
        tensors = list(k_buffers) + ([] if use_mla else list(v_buffers))
        if self._client is not None:
            self._register_with_retry(tensors, layout, group_id)

    def _register_with_retry(self, tensors, layout, group_id: int, max_retries: int = 360, delay_s: float = 1.0) -> None:
        """The transfer manager of a node other than the leader's may come up after this rank: keep trying for
        about six minutes (flexkv/integration/sglang/connector.py:1926-1950)."""
        import time
        from ...common.debug import flexkv_logger
        for attempt in range(max_retries):
            try:
                self._client.register_to_server(tensors, layout, group_id=group_id)
                return
            except Exception as e:  # noqa: BLE001
                if attempt == max_retries - 1:
                    raise
                if attempt % 30 == 0:
                    flexkv_logger.info("GPU registration retry %d/%d (tp %d pp %d): %s", attempt + 1, max_retries,
                                       self.tp_rank, self.pp_rank, e)
                time.sleep(delay_s)

    def _group_hands_off(self) -> bool:
        if self.any_hand_off is None:
            self.any_hand_off = bool(self.comm.all_reduce_min(0 if self.hand_off_slot_mapping else 1) == 0)
        return self.any_hand_off

    def _hand_off(self, task_id: Optional[int], slot_mapping: Any, n_tokens: Optional[int] = None, mask=None) -> None:
        if not self.hand_off_slot_mapping or self._client is None or task_id is None:
            return
        sm = torch.as_tensor(slot_mapping).cpu().numpy().astype(np.int64)
        if n_tokens is not None:
            sm = sm[:n_tokens]
        if mask is not None:
            sm = sm[np.asarray(mask, dtype=bool)]
        self._client.set_slot_mapping(int(task_id), sm)

    @staticmethod
    def configure_for_pool(flexkv_config: FlexKVConfig, kvcache: Any, page_size: int,
                           include_state: Optional[bool] = None) -> ResolvedPool:
        """Call BEFORE constructing the connector: reads the engine's KV pool object and, when it is made of
        several layer groups (indexer keys beside the cache, split compressed pools) or carries a
        sliding-window pool, writes the matching ``layer_groups`` / window-pool geometry into the config and
        sizes the tiers again for the new block size (flexkv/integration/sglang/connector.py:1840-1874).
        ``include_state=False`` leaves the compressor-state sidecars out of the window slot."""
        import dataclasses
        from ...common.config import recompute_block_counts
        if include_state is None:
            include_state = getattr(flexkv_config.cache_config, "_swa_multi_group", None)     # swa_multi_group key
        pool = resolve_kv_pool(kvcache, page_size, include_state)
        specs = layer_group_specs(pool, page_size)
        if specs is not None and flexkv_config.model_config.layer_groups is None:
            m = dataclasses.replace(flexkv_config.model_config, layer_groups=specs)     # the old one may be frozen
            m.freeze()
            flexkv_config.model_config = m
            recompute_block_counts(m, flexkv_config.cache_config)
        swa = window_pool_config(pool, page_size, flexkv_config.cache_config.swa)
        if swa is not None:
            flexkv_config.cache_config.swa = swa
            # the window data plane is on for such a pool unless the deployment switches it off: the geometry stays
            # configured, snapshots are neither written nor restored and every get falls back to full KV only
            # (FLEXKV_ENABLE_SWA_TRANSFER, flexkv/integration/config.py:20-21,620-627)
            flexkv_config.cache_config.enable_swa_transfer = swa_transfer_enabled_from_env()
        return pool

    def register_kv_pool(self, kvcache: Any, pool: Optional[ResolvedPool] = None) -> ResolvedPool:
        """Registers everything this rank holds of the engine's KV pool: the plain K/V (or MLA) buffers, every
        layer group of a multi-group pool, the window pages and their sidecar groups."""
        pool = pool if pool is not None else resolve_kv_pool(kvcache, self.T)
        self._kvcache = kvcache
        if not pool.multi_group:
            self.register_kv_buffers(pool.k_buffers, pool.v_buffers)
            return pool
        gid = 0
        if pool.kind == "indexer":
            self.register_kv_buffers(pool.k_buffers, pool.v_buffers, group_id=0)
            gid = 1
        for g in pool.groups:
            b0 = g.buffers[0]
            page_bytes = b0.shape[1] * b0.element_size()
            nb = self.comm.all_reduce_min(int(b0.shape[0]))
            layout = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, len(g.buffers), nb, g.sub_page_size, 1,
                                   page_bytes // g.sub_page_size, is_mla=True)
            if self._client is not None:
                self._client.register_to_server([b.view(torch.uint8) for b in g.buffers], layout, group_id=gid)
            gid += 1
        if pool.swa_buffers and self._client is not None:
            self._client.register_swa_to_server(pool.swa_buffers, group_id=0)
            for i, g in enumerate(pool.state_groups):
                self._client.register_swa_to_server(g.buffers, group_id=1 + i)
        return pool

    def _window_aware(self) -> bool:
        kvcache = getattr(self, "_kvcache", None)
        return kvcache is not None and getattr(kvcache, "swa_kv_pool", None) is not None

    def _window_page(self, slot_mapping: np.ndarray):
        """The window page of the sequence end, as the one-page slot mapping that ``launch`` binds the window
        side ops to (None: the engine keeps no window state, or the tail slid out of the window)."""
        if not self._window_aware() or len(slot_mapping) < self.T:
            return None
        m = self.swa_slot_mapping(slot_mapping)
        if m is None or len(m) < self.T:
            return None
        return [np.asarray(m[-self.T:], dtype=np.int64)]

    def swa_slot_mapping(self, full_indices: Any) -> Optional[np.ndarray]:
        """Window-pool slots for ``launch(..., swa_slot_mappings=...)``; None when the engine has no window pool
        or none of the tokens is still inside the window."""
        kvcache = getattr(self, "_kvcache", None)
        if kvcache is None:
            return None
        m = build_swa_slot_mapping(kvcache, torch.as_tensor(full_indices))
        return None if m is None else m.numpy()

    def register_layer_transfer_counter(self, kvcache: Any) -> None:
        """Installs the per-layer wait hook on SGLang's KV pool object."""
        L = self.cfg.model_config.num_layers_per_pp_stage
        self.layer_counter = FlexKVLayerDoneCounter(L, num_counters=3, world_rank=self.comm.rank)
        if hasattr(kvcache, "register_layer_transfer_counter"):
            kvcache.register_layer_transfer_counter(self.layer_counter)
        from ...transfer.layerwise import build_layerwise_eventfd_socket_path, send_eventfds
        path = build_layerwise_eventfd_socket_path(self.dp_rank, getattr(self, "pp_rank", 0), self.cfg.model_config)
        if path:
            send_eventfds(path, self.tp_rank, self.tp_size, self.layer_counter.fds_per_counter())

    def wait_ready(self, timeout: float = 600.0) -> None:
        if self.is_leader:
            self.mgr.wait_ready(timeout)
        self.comm.barrier()

    # ---- lookup / load -------------------------------------------------------------------
    # ---- two calling conventions ------------------------------------------------------------
    # The methods below take this package's arguments (request id first, lists for batches) and also the ones
    # the reference's SGLang integration passes (flexkv/integration/sglang/connector.py:460-466,696-700,956,
    # 1011-1017, as called from its sglang_flexkv_connector.patch), so that integration drives this connector
    # unchanged. Which one is meant shows in the arguments; the reference's forms return what its callers read.
    @property
    def enable_layerwise(self) -> bool:
        return bool(self.layerwise)

    def lookup_kv(self, *args: Any, **kw: Any):
        """``lookup_kv(rid, token_ids, num_computed_tokens=0, namespace=None) -> matched tokens``, or the
        reference's ``lookup_kv(token_ids, token_mask, rid=None, sglang_req_id=...) -> (task id, matched tokens)``
        where ``token_mask`` marks the tokens that are not on the GPU yet."""
        if (args and isinstance(args[0], str)) or ("token_mask" not in kw and "rid" in kw and not args):
            return self._lookup_kv(*args, **kw)
        token_ids = args[0] if args else kw["token_ids"]
        token_mask = args[1] if len(args) > 1 else kw.get("token_mask")
        rid = args[2] if len(args) > 2 else kw.get("rid")
        computed = 0
        if token_mask is not None:
            m = torch.as_tensor(token_mask).cpu().numpy().astype(bool)
            computed = int(np.argmax(m)) if m.any() else len(m)
        key = rid if rid else f"__untracked_{id(token_ids)}"
        matched = self._lookup_kv(key, token_ids, computed)
        task_id = -1
        if self.is_leader and key in self._pending_loads:
            task_id = self._pending_loads[key].task_id
        if not rid:
            self.release_pending(key)              # nobody will come back for it
        return task_id, matched

    def start_load_kv_layerwise(self, rids: Any, slot_mappings: Any):
        """Batch form ``(rids, slot_mappings) -> task ids``, or the reference's single-request form
        ``(rid, slot_mapping) -> (tokens being loaded, counter id)``."""
        if not isinstance(rids, str):
            return self._start_load_kv_layerwise(rids, slot_mappings)
        n = 0
        if self.is_leader and rids in self._pending_loads:
            n = self._pending_loads[rids].matched_tokens
        n = int(self.comm.broadcast(n))
        ids = self._start_load_kv_layerwise([rids], [slot_mappings])
        if not ids:
            return 0, -1
        producer = self.layer_counter.counter_of(ids[0]) if self.layer_counter is not None and \
            hasattr(self.layer_counter, "counter_of") else 0
        self._launched_loads.extend(ids)
        return n, producer

    def drain_launched_loads(self, task_ids: Any = 100, timeout: float = 60.0):
        """``(task_ids, timeout) -> bool`` waits for these loads; the reference's ``(threshold=100)`` is a
        non-blocking sweep over the loads launched through its single-request form, run once that many piled up."""
        if not isinstance(task_ids, int):
            return self._drain_launched_loads(task_ids, timeout)
        if len(self._launched_loads) >= task_ids:
            if self.is_leader:
                done = self.mgr.try_wait(list(dict.fromkeys(self._launched_loads)))
                self._launched_loads = [t for t in self._launched_loads if t not in done]
            else:
                self._launched_loads = []
        return None

    def store_kv(self, rid: str, token_ids: Sequence[int], slot_mapping: Any = None,
                 namespace: Optional[List[str]] = None, *, kv_indices: Any = None, sglang_req_id: Any = _UNSET):
        """Returns the tokens that will move; called the reference's way (``kv_indices=`` or ``sglang_req_id=``)
        it returns the id of the store in flight, -1 when nothing had to be stored."""
        reference_style = kv_indices is not None or sglang_req_id is not _UNSET
        moved = self._store_kv(rid, token_ids, slot_mapping if kv_indices is None else kv_indices, namespace)
        if not reference_style:
            return moved
        tid = self._stores.get(rid, -1) if self.is_leader and moved else -1
        return int(self.comm.broadcast(tid))

    def _lookup_kv(self, rid: str, token_ids: Sequence[int], num_computed_tokens: int = 0,
                   namespace: Optional[List[str]] = None) -> int:
        """Tokens beyond the GPU-resident prefix that can be restored (same on every rank)."""
        matched = 0
        if self.is_leader:
            tok = np.asarray(token_ids, dtype=np.int64)
            aligned = (len(tok) // self.T) * self.T
            if aligned > num_computed_tokens:
                mask = np.zeros(aligned, dtype=np.bool_)
                mask[num_computed_tokens:] = True
                tid, m = self.mgr.get_match(tok[:aligned], mask, namespace=namespace,
                                            swa_aware=self._window_aware())
                matched = int(m.sum())
                if matched == 0:
                    self.mgr.cancel(tid)
                else:
                    old = self._pending_loads.pop(rid, None)
                    if old is not None:
                        self.mgr.cancel(old.task_id)
                    self._pending_loads[rid] = _PendingLoad(rid, tid, matched, num_computed_tokens // self.T)
            self.stats.record_get(len(tok), num_computed_tokens, matched)
        return int(self.comm.broadcast(matched))

    def release_pending(self, rid: str) -> None:
        p = self._pending_loads.pop(rid, None)
        if p is not None and self.is_leader:
            self.mgr.cancel(p.task_id)

    def retrieve_kv(self, rid: str, slot_mapping: Any, timeout: float = 60.0) -> int:
        """Blocking load of the matched tokens into the pages named by `slot_mapping`
        (one entry per matched token). Returns the number of tokens restored."""
        done = 0
        if self._group_hands_off():
            # every rank learns the task before the leader launches it, so the other nodes can name their pages
            plan = None
            if self.is_leader:
                pl = self._pending_loads.get(rid)
                plan = (pl.task_id, pl.matched_tokens) if pl is not None else None
            plan = self.comm.broadcast(plan)
            if plan is not None:
                self._hand_off(plan[0], slot_mapping, n_tokens=plan[1])
        if self.is_leader:
            p = self._pending_loads.pop(rid, None)
            if p is not None:
                sm = torch.as_tensor(slot_mapping).cpu().numpy().astype(np.int64)[:p.matched_tokens]
                self.mgr.launch(p.task_id, sm, swa_slot_mappings=self._window_page(sm))
                rsp = self.mgr.wait(p.task_id, timeout=timeout)[p.task_id]
                done = p.matched_tokens if rsp.status == KVResponseStatus.SUCCESS else 0
                if not done:
                    self.stats.record_failed()
        return int(self.comm.broadcast(done))

    def _start_load_kv_layerwise(self, rids: Sequence[str], slot_mappings: Sequence[Any]) -> List[int]:
        """Launches the loads of a batch as ONE layerwise restore that signals per
        layer; the forward pass waits in the KV pool's layer hook."""
        ids: List[int] = []
        counter = 0
        pairs_selected = False
        if self.is_leader:
            pend = [self._pending_loads.pop(r, None) for r in rids]
            pairs = [(p, sm) for p, sm in zip(pend, slot_mappings) if p is not None]
            if pairs:
                counter = self.layer_counter.update_producer() if self.layer_counter else 0
                pairs_selected = self.layer_counter is not None
                sms = [torch.as_tensor(sm).cpu().numpy().astype(np.int64)[:p.matched_tokens] for p, sm in pairs]
                ids = self.mgr.launch([p.task_id for p, _ in pairs], sms, as_batch=True,
                                      layerwise_transfer=self.layerwise, counter_id=counter)
        manifest = self.comm.broadcast({"ids": ids, "counter": counter})
        if self.layer_counter is not None and manifest["ids"]:
            for t in manifest["ids"]:
                if self.is_leader:
                    self.layer_counter.register_task(t, manifest["counter"])
                else:
                    self.layer_counter.register_task_with_explicit_counter_id(t, manifest["counter"])
            self.layer_counter.set_consumer(manifest["ids"][0])
        elif self.layer_counter is not None and self.is_leader and pairs_selected:
            self.layer_counter.abort_unregistered_selection(counter)
        return manifest["ids"]

    def _drain_launched_loads(self, task_ids: Sequence[int], timeout: float = 60.0) -> bool:
        ok = True
        if self.is_leader and task_ids:
            res = self.mgr.wait(list(task_ids), timeout=timeout)
            ok = all(r.status == KVResponseStatus.SUCCESS for r in res.values())
        return bool(self.comm.broadcast(ok))

    # ---- store -----------------------------------------------------------------------------
    def _store_kv(self, rid: str, token_ids: Sequence[int], slot_mapping: Any,
                  namespace: Optional[List[str]] = None) -> int:
        """Asynchronous offload of the request's full pages; returns the tokens that will move."""
        moved = 0
        plan = None
        if self.is_leader:
            tok = np.asarray(token_ids, dtype=np.int64)
            aligned = (len(tok) // self.T) * self.T
            if aligned > 0:
                sm = torch.as_tensor(slot_mapping).cpu().numpy().astype(np.int64)[:aligned]
                tid, mask = self.mgr.put_match(tok[:aligned], namespace=namespace)
                moved = int(mask.sum())
                if moved == 0:
                    self.mgr.cancel(tid)
                else:
                    self.mgr.launch(tid, sm[mask], swa_slot_mappings=self._window_page(sm))
                    self._stores[rid] = tid
                    plan = (tid, aligned, np.asarray(mask, dtype=bool))
                self.stats.record_put(aligned, moved)
        if self._group_hands_off():
            plan = self.comm.broadcast(plan)
            if plan is not None:      # the other nodes' graphs wait for their pages; the order does not matter
                self._hand_off(plan[0], slot_mapping, n_tokens=plan[1], mask=plan[2])
        return int(self.comm.broadcast(moved))

    def check_completed_stores(self) -> List[str]:
        done: List[str] = []
        if self.is_leader and self._stores:
            res = self.mgr.try_wait(list(self._stores.values()))
            for rid, tid in list(self._stores.items()):
                if tid in res:
                    done.append(rid)
                    del self._stores[rid]
        return list(self.comm.broadcast(done))

    def wait_store(self, rid: str, timeout: float = 30.0) -> bool:
        ok = True
        if self.is_leader and rid in self._stores:
            tid = self._stores.pop(rid)
            ok = self.mgr.wait(tid, timeout=timeout, completely=True)[tid].status == KVResponseStatus.SUCCESS
        return bool(self.comm.broadcast(ok))

    # ---- prefetch ---------------------------------------------------------------------------
    def prefetch_async(self, rid: str, token_ids: Sequence[int], namespace: Optional[List[str]] = None,
                       sglang_req_id: Any = None) -> None:
        if not self.prefetch_enabled or not rid:
            return
        if self.is_leader:
            self._prefetch[rid] = self.mgr.prefetch_async(np.asarray(token_ids, dtype=np.int64), namespace=namespace)

    def check_prefetch_progress(self, rid: str) -> bool:
        done = True
        if self.is_leader and rid in self._prefetch:
            res = self.mgr.try_wait(self._prefetch[rid])
            done = self._prefetch[rid] in res
            if done:
                del self._prefetch[rid]
        return bool(self.comm.broadcast(done))

    def cancel_prefetch(self, rid: str) -> None:
        tid = self._prefetch.pop(rid, None)
        if tid is not None and self.is_leader:
            self.mgr.cancel(tid)

    # ---- maintenance -------------------------------------------------------------------------
    def reset(self) -> None:
        if self.is_leader:
            for p in self._pending_loads.values():
                self.mgr.cancel(p.task_id)
            self.mgr.reset()
        self._pending_loads.clear()
        self._stores.clear()
        self._prefetch.clear()
        if self.layer_counter is not None:
            self.layer_counter.reset()
        self.comm.barrier()

    def destroy(self) -> None:
        """Name used by engines that tear the connector down with the cache controller."""
        self.shutdown()

    def shutdown(self) -> None:
        if getattr(self, "_closed", False):
            return
        self._closed = True
        if self.layer_counter is not None:
            self.layer_counter.close()
        if self.is_leader and self.mgr is not None:
            try:
                self.mgr.shutdown()
            except Exception:  # noqa: BLE001
                pass
