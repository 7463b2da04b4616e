"""vLLM v1 KV-connector adapter.

``FlexKVSchedulerConnector`` lives beside vLLM's scheduler and owns a KVManager;
``FlexKVWorkerConnector`` lives in every worker and only registers that worker's
KV tensors: all data movement is done by the data plane through the shared
handles. ``FlexKVConnectorV1Impl`` is the object vLLM instantiates per role. The
contract follows the reference adapter (flexkv/integration/vllm/vllm_v1_adapter.py:
228-781 scheduler side, :783-977 worker side, :979-1283 connector):

* lookup: tokens truncated to whole blocks, mask = tokens beyond the computed
  prefix, ``get_match``; a zero hit cancels the task at once;
* bind: after allocation, the slot mapping covers only the blocks to restore;
* offload: on finish, ``put_match`` over ``((n-1)//T)*T`` tokens; if something is
  new the request's blocks stay alive until the put completes;
* step loop: cancel, launch (gets and puts batched separately), poll finished;
  failed gets report their GPU block ids so vLLM recomputes them.

Engine objects are accessed by attribute name only (request_id, all_token_ids /
prompt_token_ids, num_computed_tokens, lora_request, cache_salt ...).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import numpy as np
import torch

from ...common.debug import flexkv_logger
from ...common.request import KVResponseStatus
from ...common.storage import KVCacheLayout, KVCacheLayoutType
from ..config import FlexKVConfig
from ..stats import FlexKVStats


@dataclass
class FlexKVTask:
    task_id: int
    request_id: str
    kind: str                          # "get" | "put"
    num_tokens: int                    # tokens the task will move
    start_block: int                   # first block (in the request) the slot mapping must cover
    num_blocks: int
    slot_mapping: Optional[np.ndarray] = None
    created: float = field(default_factory=time.monotonic)
    gpu_block_ids: Optional[np.ndarray] = None
    match_start_time: float = 0.0
    match_end_time: float = 0.0
    task_launch_time: float = 0.0
    task_finished_time: float = 0.0

    @property
    def task_type(self) -> str:
        return self.kind

    @property
    def match_cost(self) -> float:
        return self.match_end_time - self.match_start_time

    @property
    def task_execute_cost(self) -> float:
        return self.task_finished_time - self.task_launch_time


def _tokens_of(request: Any) -> np.ndarray:
    for name in ("all_token_ids", "prompt_token_ids", "token_ids"):
        v = getattr(request, name, None)
        if v is not None:
            return np.asarray(list(v), dtype=np.int64)
    raise AttributeError("request has no token ids")


def _block_ids_of(blocks: Any) -> List[int]:
    """vLLM hands over KVCacheBlocks (get_block_ids() -> tuple of lists, one per group) or plain lists."""
    if blocks is None:
        return []
    if hasattr(blocks, "get_block_ids"):
        ids = blocks.get_block_ids()
        return list(ids[0]) if ids and isinstance(ids[0], (list, tuple)) else list(ids)
    if len(blocks) and isinstance(blocks[0], (list, tuple)):
        return list(blocks[0])
    return list(blocks)


def _should_offload(request: Any) -> bool:
    """A request's KV is offloaded when it finished normally (stop or length), or when it was aborted and the
    caller asked for the offload with ``offload_kv_on_finish`` (a router that moves the request elsewhere);
    any other abort leaves nothing behind (flexkv/integration/vllm/vllm_v1_adapter.py:522-532). Request
    objects that expose no finish reason count as finished normally."""
    get = getattr(request, "get_finished_reason", None)
    if get is None:
        return True
    reason = get()
    name = str(getattr(reason, "name", reason)).upper()
    if name in ("STOP", "LENGTH"):
        return True
    if name == "ABORT":
        return bool(getattr(request, "offload_kv_on_finish", False))
    return reason is None and not callable(getattr(request, "is_finished", None))


SKIP_PUT_FLAG = "/tmp/flexkv_skip_put"


class FlexKVSchedulerConnector:
    def __init__(self, flexkv_config: FlexKVConfig, kv_manager: Any = None, dp_client_id: int = 0) -> None:
        self.cfg = flexkv_config
        self.T = flexkv_config.cache_config.tokens_per_block
        if kv_manager is None:
            from ...kvmanager import KVManager
            kv_manager = KVManager(flexkv_config.model_config, flexkv_config.cache_config, dp_client_id=dp_client_id,
                                   server_recv_port=flexkv_config.server_recv_port,
                                   gpu_register_port=flexkv_config.gpu_register_port)
            kv_manager.start()
        self.mgr = kv_manager
        # operator switches (flexkv/integration/vllm/vllm_v1_adapter.py:261-264,534,1199):
        #   FLEXKV_NUM_LOG_INTERVAL_REQUESTS  hit-ratio log line every n gets (0 = never)
        #   FLEXKV_MAYBE_SKIP_PUT=1           offloads are skipped while the file SKIP_PUT_FLAG exists: a running
        #                                     deployment can be told to stop writing without a restart
        #   FLEXKV_SYNC_GET=1                 every step waits for the restores it launched (debugging aid)
        self.stats = FlexKVStats(log_interval=int(os.environ.get("FLEXKV_NUM_LOG_INTERVAL_REQUESTS", "200")))
        self.maybe_skip_put = os.environ.get("FLEXKV_MAYBE_SKIP_PUT", "0") == "1"
        self.sync_get = os.environ.get("FLEXKV_SYNC_GET", "0") == "1"
        self.req_to_get: Dict[str, FlexKVTask] = {}          # matched, waiting for allocation / launch
        self.req_to_put: Dict[str, FlexKVTask] = {}
        self.launched_get: Dict[int, FlexKVTask] = {}
        self.launched_put: Dict[int, FlexKVTask] = {}
        self.to_launch: List[FlexKVTask] = []
        self.to_cancel: List[int] = []
        self.failed_block_ids: Set[int] = set()
        self.batch_members: Dict[int, List[FlexKVTask]] = {}
        self.collector = None            # KV-cache events, see enable_kv_events()

    def enable_kv_events(self, publisher=None):
        """Buffers (or publishes) "stored" / "removed" events of the index for cache-aware routers.
        Needs the index in this process (not the client side of a separate server)."""
        eng = getattr(self.mgr, "kv_task_engine", None)
        if eng is None:
            raise RuntimeError("KV events are collected where the index lives (in-process manager or the server)")
        from ..dynamo.collector import KVEventCollector
        self.collector = KVEventCollector(publisher)
        self.collector.attach(eng.cache_engine)
        return self.collector

    # ---- lifecycle --------------------------------------------------------------------
    def is_ready(self) -> bool:
        return self.mgr.is_ready()

    def shutdown(self) -> None:
        self.mgr.shutdown()

    def reset_cache(self) -> bool:
        """After a weight update: nothing cached before may be reused."""
        self.cancel_tasks()
        self.mgr.reset()
        return True

    # ---- lookup -------------------------------------------------------------------------
    def _namespace(self, request: Any) -> Optional[List[str]]:
        ns: List[str] = []
        lora = getattr(request, "lora_request", None)
        if lora is not None:
            ns.append(str(getattr(lora, "lora_name", None) or getattr(lora, "name", lora)))
        salt = getattr(request, "cache_salt", None)
        if salt:
            ns.append(str(salt))
        extra = getattr(request, "namespace_info", None)
        if extra:
            ns.extend(str(x) for x in extra)
        return ns or None

    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int) -> Tuple[int, bool]:
        """Tokens beyond ``num_computed_tokens`` that can be restored; the bool says
        the load is asynchronous (vLLM parks the request until ``get_finished`` names it)."""
        tokens = _tokens_of(request)
        aligned = (len(tokens) // self.T) * self.T
        if aligned <= num_computed_tokens:
            return 0, False
        tokens = tokens[:aligned]
        mask = np.zeros(aligned, dtype=np.bool_)
        mask[num_computed_tokens:] = True
        task_id, matched = self.mgr.get_match(tokens, mask, namespace=self._namespace(request))
        n = int(matched.sum())
        self.stats.record_get(len(tokens), num_computed_tokens, n)
        if n == 0:
            self.mgr.cancel(task_id)
            return 0, False
        rid = str(request.request_id)
        old = self.req_to_get.pop(rid, None)
        if old is not None:
            self.to_cancel.append(old.task_id)
        self.req_to_get[rid] = FlexKVTask(task_id, rid, "get", n, num_computed_tokens // self.T, n // self.T)
        return n, True

    # ---- bind ------------------------------------------------------------------------------
    def update_state_after_alloc(self, request: Any, blocks: Any, num_external_tokens: int) -> None:
        rid = str(request.request_id)
        task = self.req_to_get.pop(rid, None)
        if task is None:
            return
        if num_external_tokens == 0:
            self.to_cancel.append(task.task_id)
            return
        ids = _block_ids_of(blocks)
        new = np.asarray(ids[task.start_block:task.start_block + task.num_blocks], dtype=np.int64)
        if len(new) < task.num_blocks:
            flexkv_logger.warning("request %s: %d blocks allocated for a %d-block restore; cancelling", rid, len(new),
                                  task.num_blocks)
            self.to_cancel.append(task.task_id)
            return
        task.gpu_block_ids = new
        task.slot_mapping = np.repeat(new, self.T) * self.T + np.tile(np.arange(self.T), len(new))
        self.to_launch.append(task)

    # ---- offload ----------------------------------------------------------------------------
    def request_finished(self, request: Any, block_ids: Sequence[int]) -> Tuple[bool, Optional[dict]]:
        """True keeps the request's blocks alive until the put completes."""
        rid = str(request.request_id)
        pending = self.req_to_get.pop(rid, None)
        if pending is not None:
            self.to_cancel.append(pending.task_id)
        if not _should_offload(request):
            return False, None
        if self.maybe_skip_put and os.path.exists(SKIP_PUT_FLAG):
            return False, None
        tokens = _tokens_of(request)
        n = ((len(tokens) - 1) // self.T) * self.T
        if n <= 0:
            return False, None
        tokens = tokens[:n]
        task_id, mask = self.mgr.put_match(tokens, namespace=self._namespace(request))
        new = int(mask.sum())
        self.stats.record_put(n, new)
        if new == 0:
            self.mgr.cancel(task_id)
            return False, None
        first = int(np.flatnonzero(mask)[0]) // self.T
        ids = np.asarray(list(block_ids)[first:first + new // self.T], dtype=np.int64)
        if len(ids) < new // self.T:
            self.mgr.cancel(task_id)
            return False, None
        task = FlexKVTask(task_id, rid, "put", new, first, new // self.T, gpu_block_ids=ids)
        task.slot_mapping = np.repeat(ids, self.T) * self.T + np.tile(np.arange(self.T), len(ids))
        self.to_launch.append(task)
        return True, None

    # ---- step loop --------------------------------------------------------------------------
    def cancel_tasks(self) -> None:
        for t in self.req_to_get.values():
            self.to_cancel.append(t.task_id)
        self.req_to_get.clear()
        if self.to_cancel:
            self.mgr.cancel(self.to_cancel)
            self.to_cancel = []

    def flush_cancels(self) -> None:
        if self.to_cancel:
            self.mgr.cancel(self.to_cancel)
            self.to_cancel = []

    def launch_tasks(self) -> None:
        gets = [t for t in self.to_launch if t.kind == "get"]
        puts = [t for t in self.to_launch if t.kind == "put"]
        self.to_launch = []
        for group, book in ((gets, self.launched_get), (puts, self.launched_put)):
            if not group:
                continue
            ids = self.mgr.launch([t.task_id for t in group], [t.slot_mapping for t in group], as_batch=len(group) > 1)
            if len(ids) == 1 and len(group) > 1:
                self.batch_members[ids[0]] = group
                book[ids[0]] = group[0]
            else:
                for t in group:
                    book[t.task_id] = t

    def query_finished_task(self) -> Tuple[Set[str], Set[str]]:
        """(request ids whose put finished, request ids whose get finished)."""
        sending, recving = set(), set()
        for book, out, is_get in ((self.launched_put, sending, False), (self.launched_get, recving, True)):
            if not book:
                continue
            done = self.mgr.try_wait(list(book))
            for tid, rsp in done.items():
                members = self.batch_members.pop(tid, None) or [book[tid]]
                book.pop(tid, None)
                for t in members:
                    out.add(t.request_id)
                    if rsp.status != KVResponseStatus.SUCCESS:
                        self.stats.record_failed()
                        if is_get and t.gpu_block_ids is not None:
                            self.failed_block_ids.update(int(b) for b in t.gpu_block_ids)
        return sending, recving

    def _blocking_wait(self, book: Dict[int, FlexKVTask], timeout: float = 120.0) -> List[Any]:
        """Waits for every launched task of ``book``; used at engine shutdown and by synchronous callers."""
        out: List[Any] = []
        ids = list(book)
        if not ids:
            return out
        done = self.mgr.wait(ids, timeout=timeout, completely=True)
        for tid, rsp in done.items():
            book.pop(tid, None)
            self.batch_members.pop(tid, None)
            out.append(rsp)
        return out

    def wait_for_all_get_tasks(self) -> List[Any]:
        self.launch_tasks()
        return self._blocking_wait(self.launched_get)

    def wait_for_all_put_tasks(self) -> List[Any]:
        self.launch_tasks()
        return self._blocking_wait(self.launched_put)

    def get_and_clear_failed_block_ids(self) -> Set[int]:
        out, self.failed_block_ids = self.failed_block_ids, set()
        return out

    def handle_preemptions(self, preempted_req_ids: Iterable[str]) -> None:
        """Unlaunched work of a preempted request is dropped; launched transfers run to completion."""
        gone = {str(r) for r in preempted_req_ids}
        for rid in list(self.req_to_get):
            if rid in gone:
                self.to_cancel.append(self.req_to_get.pop(rid).task_id)
        keep = []
        for t in self.to_launch:
            if t.request_id in gone:
                self.to_cancel.append(t.task_id)
            else:
                keep.append(t)
        self.to_launch = keep

    def wait_for_all(self, timeout: float = 60.0) -> None:
        ids = list(self.launched_get) + list(self.launched_put)
        if ids:
            self.mgr.wait(ids, timeout=timeout, completely=True)


def infer_vllm_gpu_layout(kv_caches: Sequence[torch.Tensor], tokens_per_block: int, num_kv_heads: int, head_size: int,
                          use_mla: bool) -> KVCacheLayout:
    """Tells the two vLLM cache shapes apart by inspecting the real tensor:
    flash-attn ``[2, N, T, H, D]`` vs flashinfer / triton ``[N, 2, T, H, D]``; MLA is
    ``[N, T, D]``; packed single-region caches are ``[N, H, T, W]`` (flexkv/integration/vllm/vllm_v1_adapter.py:846-905)."""
    t = kv_caches[0]
    L = len(kv_caches)
    if use_mla or t.dim() == 3:
        return KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, t.shape[0], tokens_per_block, 1, t.shape[-1], is_mla=True)
    if t.dim() == 4:
        # packed caches without a K/V axis: (blocks, H, tokens, 2 * D), or FlashInfer NVFP4 (blocks, 2 * H,
        # tokens, D packed). One region per block and layer; the chunk moves whole, so the order of heads and
        # tokens inside it is the engine's business (flexkv/integration/vllm/vllm_v1_adapter.py:852-874)
        return KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, t.shape[0], t.shape[2], t.shape[1], t.shape[3],
                             is_mla=True)
    if t.dim() != 5:
        raise ValueError(f"unsupported vLLM KV cache shape {tuple(t.shape)}")
    if t.shape[0] == 2 and t.shape[1] != 2:
        ltype, nb = KVCacheLayoutType.LAYERFIRST, t.shape[1]
    elif t.shape[1] == 2:
        ltype, nb = KVCacheLayoutType.LAYERBLOCK, t.shape[0]
    else:
        ltype, nb = KVCacheLayoutType.LAYERFIRST, t.shape[1]
    return KVCacheLayout(ltype, L, nb, t.shape[2], t.shape[3], t.shape[4])


class FlexKVWorkerConnector:
    def __init__(self, flexkv_config: FlexKVConfig, dp_client_id: int = 0, tp_rank: int = 0, pp_rank: int = 0,
                 device_id: Optional[int] = None) -> None:
        from ...server.client import KVTPClient
        self.cfg = flexkv_config
        self.device_id = torch.cuda.current_device() if device_id is None and torch.cuda.is_available() else (device_id or 0)
        self.client = KVTPClient(flexkv_config.gpu_register_port, dp_client_id, self.device_id, tp_rank=tp_rank,
                                 pp_rank=pp_rank)
        self._caches: Optional[List[torch.Tensor]] = None
        self._layout: Optional[KVCacheLayout] = None

    def _split(self, kv_caches) -> List[Tuple[str, List[torch.Tensor], List[int]]]:
        """The worker's tensors as ordered groups ``(kind, tensors, layer ids)``. Layers that share one tensor
        (the same storage under several layer names) count once. Attention caches are grouped by shape and
        dtype in order of first appearance: a model whose sliding-window layers and full-attention layers have
        different head counts or head sizes yields one group per shape. Tensors whose layer name contains
        ``.k_cache`` are indexer key caches and form the last group."""
        named = kv_caches if isinstance(kv_caches, dict) else {str(i): t for i, t in enumerate(kv_caches)}
        seen, main, indexer = set(), [], []
        for name, t in named.items():
            key = (t.data_ptr(), tuple(t.shape)) if t.numel() else id(t)
            if key in seen:
                continue
            seen.add(key)
            (indexer if ".k_cache" in name else main).append(t)
        groups: Dict[Any, Tuple[List[torch.Tensor], List[int]]] = {}
        for i, t in enumerate(main):
            ts, ids = groups.setdefault((tuple(t.shape), t.dtype), ([], []))
            ts.append(t)
            ids.append(i)
        out = [("kv", ts, ids) for ts, ids in groups.values()]
        if indexer:
            out.append(("indexer", indexer, list(range(len(indexer)))))
        return out

    def register_to_server(self, kv_caches: Dict[str, torch.Tensor]) -> None:
        """Registers the worker's KV tensors. One shape: a plain registration. Several shapes (layers with
        different head geometry, indexer key caches ``[blocks, tokens, dim]`` beside the attention layers): one
        layer group per shape, and the group list travels with the registration because only the worker sees
        these tensors (flexkv/integration/vllm/vllm_v1_adapter.py:826-960)."""
        m, c = self.cfg.model_config, self.cfg.cache_config
        parts = self._split(kv_caches)
        regs: List[Tuple[List[torch.Tensor], KVCacheLayout]] = []
        for kind, ts, _ in parts:
            if kind == "indexer":
                t0 = ts[0]
                if t0.dim() != 3:
                    raise ValueError(f"indexer caches are [blocks, tokens, dim], got {tuple(t0.shape)}")
                regs.append((ts, KVCacheLayout(KVCacheLayoutType.LAYERFIRST, len(ts), t0.shape[0], t0.shape[1], 1,
                                               t0.shape[2], is_mla=True)))
            else:
                regs.append((ts, infer_vllm_gpu_layout(ts, c.tokens_per_block, m.num_kv_heads // max(1, m.tp_size),
                                                       m.head_size, m.use_mla)))
        self._caches, self._layout = regs[0]
        self._regs = regs
        if len(regs) == 1:
            self.client.register_to_server(*regs[0])
            return
        from ...common.config import LayerGroupSpec
        T = regs[0][1].tokens_per_block
        groups = []
        for gi, ((kind, ts, ids), (_, lay)) in enumerate(zip(parts, regs)):
            groups.append(LayerGroupSpec(
                num_layers=len(ts), num_kv_heads=lay.num_head, head_size=lay.head_size, kv_dim=lay.kv_dim,
                dtype=ts[0].dtype, layer_ids=list(ids), name=kind if kind == "indexer" else f"kv{gi}" if gi else "kv",
                compress_ratio=max(1, T // int(lay.tokens_per_block)) if kind == "indexer" else 1))
        self._groups = groups
        for gi, (ts, lay) in enumerate(regs):
            self.client.register_to_server(ts, lay, group_id=gi, layer_groups=groups)

    def before_device_sleep(self) -> int:
        """vLLM sleep mode frees the cache; the data plane must stop touching (and mapping) it first.
        The host tier is kept. Returns 0 when the data plane confirmed."""
        return 0 if self.client.suspend_gpu_mappings() else 1

    def after_device_wake(self, kv_caches: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """Pass the re-created tensors when the engine allocated a new cache on wake."""
        regs = getattr(self, "_regs", None)
        if not regs:
            return
        if kv_caches is not None:
            parts = self._split(kv_caches)
            if [len(ts) for _, ts, _ in parts] != [len(ts) for ts, _ in regs]:
                raise ValueError("the cache that came back after wake has a different set of tensors")
            regs = self._regs = [(ts, lay) for (_, ts, _), (_, lay) in zip(parts, regs)]
            self._caches = regs[0][0]
        if len(regs) == 1:
            self.client.resume_gpu_mappings(regs[0][0], regs[0][1])
        else:
            self.client.resume_gpu_mappings(regs[0][0], regs[0][1], group_id=0,
                                            more_groups=[(ts, lay, gi) for gi, (ts, lay) in enumerate(regs) if gi])


_VLLM_TYPES: Optional[dict] = None


class _PlainConnectorMetadata:
    """Stand-in for the step record where vLLM is not importable (tests with fake engine objects)."""

    def __init__(self, finished_sending=(), finished_recving=()) -> None:
        self.finished_sending = set(finished_sending)
        self.finished_recving = set(finished_recving)

    def __getitem__(self, key):
        return {"finished_sending": self.finished_sending, "finished_recving": self.finished_recving}[key]


def _vllm_types() -> dict:
    """vLLM's own metadata and stats base classes when vLLM is importable (its scheduler and logger check the
    types of what a connector returns), plain stand-ins otherwise. Resolved once, on first use."""
    global _VLLM_TYPES
    if _VLLM_TYPES is None:
        try:
            from . import vllm_types as vt
            _VLLM_TYPES = dict(meta=vt.FlexKVConnectorMetadata, stats=vt.FlexKVConnectorStats,
                               worker_stats=vt.FlexKVWorkerSentinelStats)
        except Exception:  # noqa: BLE001 - no vLLM here
            _VLLM_TYPES = dict(meta=_PlainConnectorMetadata, stats=None, worker_stats=None)
    return _VLLM_TYPES


class FlexKVConnectorV1Impl:
    """Role-dispatching object behind vLLM's ``KVConnectorBase_V1`` interface."""

    def __init__(self, vllm_config: Any, role: Any) -> None:
        self.cfg = FlexKVConfig.from_env()
        self.cfg.post_init_from_vllm_config(vllm_config)
        role_name = str(getattr(role, "name", role)).upper()
        self.is_scheduler = "SCHEDULER" in role_name
        pc = getattr(vllm_config, "parallel_config", None)
        dp_rank = int(getattr(pc, "data_parallel_rank", 0) or 0)
        if self.is_scheduler:
            self.scheduler = FlexKVSchedulerConnector(self.cfg, dp_client_id=dp_rank)
            self.worker = None
        else:
            tp_rank = int(getattr(pc, "rank", 0) or 0) % max(1, self.cfg.model_config.tp_size)
            self.worker = FlexKVWorkerConnector(self.cfg, dp_client_id=dp_rank, tp_rank=tp_rank)
            self.scheduler = None
        self._finished_sending: Set[str] = set()
        self._finished_recving: Set[str] = set()
        self._previous_scheduled: Set[str] = set()

    # worker side: data moves outside the forward pass, so these hooks are no-ops
    def start_load_kv(self, forward_context: Any, **kw: Any) -> None: ...
    def wait_for_layer_load(self, layer_name: str) -> None: ...
    def save_kv_layer(self, layer_name: str, kv_layer: torch.Tensor, attn_metadata: Any, **kw: Any) -> None: ...
    def wait_for_save(self) -> None: ...

    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]) -> None:
        self.worker.register_to_server(kv_caches)

    # sleep mode: the engine releases (and later re-creates) its cache memory around these two calls
    # (flexkv/integration/vllm/vllm_v1_adapter.py:1115-1125); a scheduler-role object has nothing to do
    def before_device_sleep(self) -> None:
        if self.worker is not None:
            self.worker.before_device_sleep()

    def after_device_wake(self, kv_caches: Optional[Dict[str, torch.Tensor]] = None) -> None:
        if self.worker is not None:
            self.worker.after_device_wake(kv_caches)

    def get_finished(self, finished_req_ids: Set[str]) -> Tuple[Optional[Set[str]], Optional[Set[str]]]:
        s, r = self._finished_sending, self._finished_recving
        self._finished_sending, self._finished_recving = set(), set()
        return s or None, r or None

    # scheduler side
    def get_num_new_matched_tokens(self, request: Any, num_computed_tokens: int) -> Tuple[int, bool]:
        return self.scheduler.get_num_new_matched_tokens(request, num_computed_tokens)

    def update_state_after_alloc(self, request: Any, blocks: Any, num_external_tokens: int) -> None:
        self.scheduler.update_state_after_alloc(request, blocks, num_external_tokens)

    def build_connector_meta(self, scheduler_output: Any):
        s = self.scheduler
        pre = getattr(scheduler_output, "preempted_req_ids", None)
        if pre is None:
            # engines whose scheduler output does not name the preempted requests: whoever was scheduled in the
            # last step, is not scheduled now and did not finish was preempted
            now = {getattr(r, "req_id", None) for r in (getattr(scheduler_output, "scheduled_new_reqs", None) or [])}
            cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
            now.update(getattr(cached, "req_ids", None) or [])
            now.discard(None)
            done = set(getattr(scheduler_output, "finished_req_ids", None) or [])
            pre = self._previous_scheduled - now - done
            self._previous_scheduled = now
        if pre:
            s.handle_preemptions(pre)
        s.flush_cancels()
        s.launch_tasks()
        sending, recving = s.query_finished_task()
        if s.sync_get:
            # the step does not return before the restores it launched have landed; they are reported as
            # finished through the same sets as in the asynchronous case
            deadline = time.monotonic() + 120.0
            while s.launched_get and time.monotonic() < deadline:
                time.sleep(0.0005)
                more_s, more_r = s.query_finished_task()
                sending |= more_s
                recving |= more_r
        # finished transfers reach the engine through update_connector_output (below); engines that read the
        # step record instead get them there as well
        self._finished_sending |= set(sending)
        self._finished_recving |= set(recving)
        return _vllm_types()["meta"](sending, recving)

    def update_connector_output(self, connector_output: Any) -> None:
        """Scheduler side, once per step after the model runner's output came back: the requests whose offload
        or restore has finished are written into the engine's connector output, which is what releases a
        finished request's pages and resumes a request that waited for its restore
        (reference: flexkv/integration/vllm/vllm_v1_adapter.py:1204-1220)."""
        if not self.is_scheduler or connector_output is None:
            return
        sending, recving = self.scheduler.query_finished_task()
        sending = set(sending) | self._finished_sending
        recving = set(recving) | self._finished_recving
        self._finished_sending, self._finished_recving = set(), set()
        for name, got in (("finished_sending", sending), ("finished_recving", recving)):
            have = getattr(connector_output, name, None)
            merged = (set(have) if have else set()) | got
            setattr(connector_output, name, merged if merged else have)

    def request_finished(self, request: Any, block_ids: Sequence[int]) -> Tuple[bool, Optional[dict]]:
        return self.scheduler.request_finished(request, block_ids)

    def take_events(self) -> List[Any]:
        """Buffered KV-cache events (stored / removed) for routers that track cache contents."""
        col = getattr(self.scheduler, "collector", None) if self.scheduler else None
        if col is None:
            return []
        from ..dynamo.collector import to_vllm_events
        return to_vllm_events(col.take_events(), self.scheduler.T)

    def get_kv_connector_stats(self) -> Optional[dict]:
        """Counters of the last interval. The worker side returns an empty (non-None) record so that the
        engine keeps polling for finished transfers on steps that schedule no tokens."""
        types = _vllm_types()
        cls = types["stats"]
        if not self.is_scheduler:
            sentinel = types.get("worker_stats")
            return {} if sentinel is None else sentinel(data={})
        st = self.scheduler.stats
        total = dict(num_get_requests=st.num_get_requests, num_get_query_tokens=st.num_get_query_tokens,
                     num_gpu_matched_tokens=st.num_gpu_matched_tokens,
                     num_flexkv_matched_tokens=st.num_flexkv_matched_tokens, num_put_requests=st.num_put_requests,
                     num_put_query_tokens=st.num_put_query_tokens,
                     num_put_unmatched_tokens=st.num_put_unmatched_tokens, num_failed_requests=st.num_failed_requests)
        # the engine's logger ADDS the records of an interval: hand over what happened since the last call
        last = getattr(self, "_stats_reported", {})
        d = {k: v - last.get(k, 0) for k, v in total.items()}
        self._stats_reported = total
        return d if cls is None else cls(data=d)

    def get_block_ids_with_load_errors(self) -> Set[int]:
        return self.scheduler.get_and_clear_failed_block_ids() if self.scheduler else set()

    def reset_cache(self) -> Optional[bool]:
        return self.scheduler.reset_cache() if self.scheduler else None

    def shutdown(self) -> None:
        if self.scheduler:
            self.scheduler.shutdown()
