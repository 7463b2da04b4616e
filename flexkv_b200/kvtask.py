"""Task layer: turns API calls into planned transfer graphs, tracks them to
completion and maps the outcome to ``KVResponse``.

Behavioural counterpart of the reference's KVTaskManager / KVTaskEngine
(flexkv/kvtask.py:40-113 task states, :305-425 task creation, :450-555
completion drain, :712-776 failure / end-op semantics, :879-986 aggregation
over several transfer handles, :988-1488 engine API). Semantics kept:

* ``get_match`` / ``put_match`` plan without GPU block ids; ``launch`` binds
  the slot mapping (one id per block: ``slot_mapping[::T] // T``) and submits;
* ``wait(..., completely=False)`` returns when the task's *end op* is done (a
  put reports success after the GPU->host copy, possibly before the SSD write);
* an op failure makes the task FAILED (never TIMEOUT) after all in-flight ops of
  its graph drained, and its plan is aborted: locks released, unready index
  nodes rolled back, staging blocks returned;
* matching calls first drain completions so finished copies are visible.
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import numpy as np

from .cache.cache_engine import GlobalCacheEngine, TransferPlanHandle, slot_mapping_to_block_ids
from .common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from .common.debug import flexkv_logger, log_op
from .common.request import KVResponse, KVResponseStatus
from .common.tracer import FlexKVTracer
from .common.transfer import CompletedOp, TransferOpGraph, merge_to_batch_graph
from .utils import nvtx_range


class TaskStatus(Enum):
    UNREADY = "unready"        # planned, GPU blocks not bound yet
    READY = "ready"            # bound, not submitted
    RUNNING = "running"
    COMPLETED = "completed"
    CANCELLED = "cancelled"
    FAILED = "failed"


class TaskType(Enum):
    GET = "get"
    PUT = "put"
    PREFETCH = "prefetch"
    BATCH_GET = "batch_get"
    BATCH_PUT = "batch_put"


_STATUS_MAP = {TaskStatus.COMPLETED: KVResponseStatus.SUCCESS, TaskStatus.CANCELLED: KVResponseStatus.CANCELLED,
               TaskStatus.FAILED: KVResponseStatus.FAILED}


@dataclass
class KVTask:
    task_id: int
    task_type: TaskType
    token_ids: Optional[np.ndarray]
    token_mask: Optional[np.ndarray]
    slot_mapping: Optional[np.ndarray]
    dp_id: int
    graph: TransferOpGraph
    return_mask: Optional[Union[np.ndarray, List[np.ndarray]]]
    plan_handle: Optional[TransferPlanHandle]
    op_callback_dict: Dict[int, Callable]
    task_end_op_id: int
    status: TaskStatus = TaskStatus.UNREADY
    task_end_op_finished: bool = False
    children: List[int] = field(default_factory=list)     # batch task -> member task ids
    parent: int = -1
    op_remap: Dict[int, int] = field(default_factory=dict)
    handles_pending: int = 0
    any_failed: bool = False
    created_at: float = field(default_factory=time.monotonic)
    failed_gpu_blocks: Optional[np.ndarray] = None

    def is_completed(self) -> bool:
        return self.status in (TaskStatus.COMPLETED, TaskStatus.CANCELLED, TaskStatus.FAILED)

    def shed_heavy_resources(self) -> None:
        """A finished task is kept until its answer was fetched (or its time-to-live ran out); what it no longer
        needs - token ids, slot mapping, the op graph, callbacks - goes at once, status and return mask stay
        (flexkv/kvtask.py:106-113)."""
        self.graph = None
        self.token_ids = self.token_mask = self.slot_mapping = None
        self.op_callback_dict = {}
        self.op_remap = {}


class ExpiringDict(OrderedDict):
    """Insertion-ordered dict that forgets entries older than ``ttl`` seconds or
    beyond ``max_len`` (abandoned tasks must not leak; flexkv/kvtask.py:212)."""

    def __init__(self, ttl: float = 1800.0, max_len: int = 100000) -> None:
        super().__init__()
        self.ttl, self.max_len = ttl, max_len
        self._stamp: Dict[Any, float] = {}

    def __setitem__(self, k, v) -> None:
        super().__setitem__(k, v)
        self._stamp[k] = time.monotonic()
        self._prune()

    def __delitem__(self, k) -> None:
        super().__delitem__(k)
        self._stamp.pop(k, None)

    def _prune(self) -> None:
        now = time.monotonic()
        while self and (len(self) > self.max_len or now - self._stamp[next(iter(self))] > self.ttl):
            k = next(iter(self))
            v = self[k]
            if isinstance(v, KVTask) and v.status == TaskStatus.RUNNING and len(self) <= self.max_len:
                break       # never forget a transfer that is still in flight
            del self[k]


class KVTaskEngine:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig,
                 transfer_handles: Optional[List[Any]] = None, cache_engine: Optional[GlobalCacheEngine] = None,
                 storage: Any = None) -> None:
        self.model_config = model_config
        self.cache_config = cache_config
        self.cache_engine = cache_engine or GlobalCacheEngine(cache_config, model_config)
        self.storage = storage
        self.transfer_handles: List[Any] = list(transfer_handles or [])
        self.tasks: ExpiringDict = ExpiringDict(ttl=GLOBAL_CONFIG_FROM_ENV.task_ttl_seconds)
        self.graph_to_task: Dict[int, int] = {}
        self._op_reports: Dict[Tuple[int, int], list] = {}     # (graph, op) -> reports so far, several handles only
        self._task_id = 0
        self._lock = threading.RLock()
        self._epoch = 0                      # bumped by reset_cache; stale completions are neutered
        self.tracer = FlexKVTracer.from_env(model_config, cache_config)
        self._metrics = None

    # ---- lifecycle ------------------------------------------------------------
    def start(self) -> None:
        for h in self.transfer_handles:
            h.start()

    def is_ready(self) -> bool:
        return all(h.is_ready() for h in self.transfer_handles)

    def shutdown(self) -> None:
        for h in self.transfer_handles:
            h.shutdown()
        self.cache_engine.shutdown()
        self.tracer.close()

    def set_metrics_collector(self, collector) -> None:
        self._metrics = collector
        self.cache_engine.set_metrics_collector(collector)
        for h in self.transfer_handles:
            if hasattr(h, "set_metrics_collector"):
                h.set_metrics_collector(collector)

    def _gen_task_id(self) -> int:
        with self._lock:
            self._task_id += 1
            return self._task_id - 1

    # ---- creation -------------------------------------------------------------
    def _new_task(self, task_type: TaskType, token_ids, token_mask, slot_mapping, dp_id, planned) -> KVTask:
        graph, mask, handle, cbs, end_op = planned
        tid = self._gen_task_id()
        task = KVTask(tid, task_type, token_ids, token_mask, slot_mapping, dp_id, graph, mask, handle, cbs, end_op)
        if graph.num_ops == 0:
            # nothing to move: the task is complete on creation
            task.status = TaskStatus.COMPLETED
            task.task_end_op_finished = True
            handle.complete()
        elif graph.gpu_bound:
            task.status = TaskStatus.READY
        graph.task_id = tid         # the name other nodes of the group know the task by (slot-mapping hand-off)
        with self._lock:
            self.tasks[tid] = task
            self.graph_to_task[graph.graph_id] = tid
        return task

    def _create_get(self, token_ids, token_mask, slot_mapping, dp_id, namespace, cpu_only=False,
                    swa_aware=False) -> KVTask:
        with nvtx_range("flexkv.get.plan"):
            planned = self.cache_engine.get(-1, token_ids, token_mask, slot_mapping, dp_id, namespace,
                                            cpu_only=cpu_only, swa_aware=swa_aware)
        return self._new_task(TaskType.GET, token_ids, token_mask, slot_mapping, dp_id, planned)

    def _create_put(self, token_ids, token_mask, slot_mapping, dp_id, namespace) -> KVTask:
        with nvtx_range("flexkv.put.plan"):
            planned = self.cache_engine.put(-1, token_ids, token_mask, slot_mapping, dp_id, namespace)
        return self._new_task(TaskType.PUT, token_ids, token_mask, slot_mapping, dp_id, planned)

    # names of the reference's task manager for the same steps (flexkv/kvtask.py:305-425)
    def create_get_task(self, token_ids, token_mask=None, slot_mapping=None, dp_id: int = 0, namespace=None,
                        cpu_only: bool = False, swa_aware: bool = False) -> KVTask:
        return self._create_get(token_ids, token_mask, slot_mapping, dp_id, namespace, cpu_only, swa_aware)

    def create_put_task(self, token_ids, token_mask=None, slot_mapping=None, dp_id: int = 0, namespace=None) -> KVTask:
        return self._create_put(token_ids, token_mask, slot_mapping, dp_id, namespace)

    def check_completed(self, task_id: int) -> bool:
        self._update_tasks(timeout=0)
        t = self.tasks.get(task_id)
        return t is None or t.status in (TaskStatus.COMPLETED, TaskStatus.CANCELLED, TaskStatus.FAILED)

    def check_task_ready(self, task_id: int) -> bool:
        t = self.tasks.get(task_id)
        return t is not None and t.status != TaskStatus.UNREADY

    # ---- API ------------------------------------------------------------------
    def get_async(self, token_ids: np.ndarray, slot_mapping: np.ndarray, token_mask: Optional[np.ndarray] = None,
                  dp_id: int = 0, namespace: Optional[List[str]] = None) -> Tuple[int, np.ndarray]:
        self._update_tasks(timeout=0)
        task = self._create_get(token_ids, token_mask, slot_mapping, dp_id, namespace)
        self.tracer.trace_request("GET", task.task_id, token_ids, slot_mapping, token_mask, namespace)
        task.graph.set_swa_pages(None)      # the one-call API carries no window pages
        self._launch([task])
        return task.task_id, task.return_mask

    def put_async(self, token_ids: np.ndarray, slot_mapping: np.ndarray, token_mask: Optional[np.ndarray] = None,
                  dp_id: int = 0, namespace: Optional[List[str]] = None) -> Tuple[int, np.ndarray]:
        self._update_tasks(timeout=0)
        task = self._create_put(token_ids, token_mask, slot_mapping, dp_id, namespace)
        self.tracer.trace_request("PUT", task.task_id, token_ids, slot_mapping, token_mask, namespace)
        task.graph.set_swa_pages(None)
        self._launch([task])
        return task.task_id, task.return_mask

    def get_match(self, token_ids: np.ndarray, token_mask: Optional[np.ndarray] = None, dp_id: int = 0,
                  cpu_only: bool = False, namespace: Optional[List[str]] = None, swa_aware: bool = False
                  ) -> Tuple[int, np.ndarray]:
        self._update_tasks(timeout=0)
        task = self._create_get(token_ids, token_mask, None, dp_id, namespace, cpu_only=cpu_only, swa_aware=swa_aware)
        self.tracer.trace_request("GET_MATCH", task.task_id, token_ids, None, token_mask, namespace)
        return task.task_id, task.return_mask

    def put_match(self, token_ids: np.ndarray, token_mask: Optional[np.ndarray] = None, dp_id: int = 0,
                  namespace: Optional[List[str]] = None) -> Tuple[int, np.ndarray]:
        self._update_tasks(timeout=0)
        task = self._create_put(token_ids, token_mask, None, dp_id, namespace)
        self.tracer.trace_request("PUT_MATCH", task.task_id, token_ids, None, token_mask, namespace)
        return task.task_id, task.return_mask

    def prefetch_async(self, token_ids: np.ndarray, dp_id: int = 0, namespace: Optional[List[str]] = None,
                       swa_aware: bool = False) -> int:
        """Pulls the SSD / remote part of a prefix into the host pool ahead of
        scheduling; the response mask marks the tokens that became host-resident."""
        self._update_tasks(timeout=0)
        planned = self.cache_engine.get(-1, token_ids, None, None, dp_id, namespace, prefetch=True)
        task = self._new_task(TaskType.PREFETCH, token_ids, None, None, dp_id, planned)
        self.tracer.trace_request("PREFETCH", task.task_id, token_ids, None, None, namespace)
        self._launch([task])
        return task.task_id

    def launch_tasks(self, task_ids: List[int], slot_mappings: List[np.ndarray], swa_slot_mappings=None,
                     as_batch: bool = False, batch_id: int = -1, layerwise_transfer: bool = False,
                     counter_id: int = 0) -> List[int]:
        if len(task_ids) != len(slot_mappings):
            raise ValueError("one slot mapping per task is required")
        self.tracer.trace_launch(task_ids, slot_mappings, as_batch, layerwise_transfer, counter_id)
        tasks: List[KVTask] = []
        with self._lock:
            for i, (tid, sm) in enumerate(zip(task_ids, slot_mappings)):
                task = self.tasks.get(tid)
                if task is None:
                    raise KeyError(f"unknown task {tid}")
                if task.status == TaskStatus.UNREADY:
                    ids = slot_mapping_to_block_ids(np.asarray(sm, dtype=np.int64), self.cache_config.tokens_per_block)
                    task.graph.set_gpu_blocks(ids)
                    # window side ops: one page of window slots per task, or none (side ops become no-ops)
                    swa_sm = swa_slot_mappings[i] if swa_slot_mappings is not None and i < len(swa_slot_mappings) \
                        else None
                    task.graph.set_swa_pages(None if swa_sm is None else slot_mapping_to_block_ids(
                        np.asarray(swa_sm, dtype=np.int64), self.cache_config.tokens_per_block))
                    task.slot_mapping = sm
                    task.status = TaskStatus.READY
                tasks.append(task)
        live = [t for t in tasks if t.status == TaskStatus.READY]
        all_get = all(t.task_type == TaskType.GET for t in live)
        all_put = all(t.task_type == TaskType.PUT for t in live)
        if layerwise_transfer and not all_get:
            flexkv_logger.warning("layerwise transfer serves gets only; falling back to a plain launch")
            layerwise_transfer = False
        if live and as_batch and (len(live) > 1 or layerwise_transfer) and (all_get or all_put):
            bid = self._merge_to_batch(live, TaskType.BATCH_GET if all_get else TaskType.BATCH_PUT, batch_id,
                                       layerwise_transfer, counter_id)
            return [bid]
        self._launch(live)
        return list(task_ids)

    def _merge_to_batch(self, members: List[KVTask], ttype: TaskType, batch_id: int, layerwise: bool,
                        counter_id: int) -> int:
        merged, remap = merge_to_batch_graph([t.graph for t in members], layerwise=layerwise, counter_id=counter_id)
        bid = batch_id if batch_id >= 0 else self._gen_task_id()
        batch = KVTask(bid, ttype, None, None, None, members[0].dp_id, merged,
                       [t.return_mask for t in members], None, {}, -1, status=TaskStatus.READY)
        batch.children = [t.task_id for t in members]
        batch.op_remap = remap
        # the batch ends (for wait(completely=False)) when the images of all members' end ops are done
        ends = sorted({remap[t.task_end_op_id] for t in members if t.task_end_op_id in remap})
        if len(ends) == 1:
            batch.task_end_op_id = ends[0]
        elif ends:
            batch.task_end_op_id = merged.add_virtual_op(ends)
        with self._lock:
            for t in members:
                t.parent = bid
                t.status = TaskStatus.RUNNING
                self.graph_to_task.pop(t.graph.graph_id, None)
            merged.task_id = bid
            self.tasks[bid] = batch
            self.graph_to_task[merged.graph_id] = bid
        self._launch([batch])
        return bid

    def _launch(self, tasks: List[KVTask]) -> None:
        graphs = []
        with self._lock:
            for t in tasks:
                if t.status != TaskStatus.READY:
                    continue
                t.status = TaskStatus.RUNNING
                t.handles_pending = len(self.transfer_handles)
                graphs.append(t.graph)
        if not graphs:
            return
        with nvtx_range("flexkv.launch"):
            for h in self.transfer_handles:
                h.submit_batch(graphs)
        for t in tasks:
            log_op(t.task_type.value, "launch", "ok", task_id=t.task_id, ops=t.graph.num_ops)

    def cancel_tasks(self, task_ids: Union[int, List[int]]) -> None:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        with self._lock:
            for tid in task_ids:
                task = self.tasks.get(tid)
                if task is None or task.is_completed():
                    continue
                if task.status == TaskStatus.RUNNING:
                    flexkv_logger.warning("task %d is already running and cannot be cancelled", tid)
                    continue
                task.status = TaskStatus.CANCELLED
                if task.plan_handle is not None:
                    task.plan_handle.abort()
                self.graph_to_task.pop(task.graph.graph_id, None)
                log_op(task.task_type.value, "cancel", "ok", task_id=tid)

    # ---- completion -----------------------------------------------------------
    def _update_tasks(self, timeout: float = 0.0) -> None:
        """Drains completions from every transfer handle and advances task state."""
        per_handle = timeout / max(1, len(self.transfer_handles)) if timeout else 0.0
        if len(self.transfer_handles) == 1:
            for c in self.transfer_handles[0].wait(timeout=per_handle):
                self._on_completed(c)
            return
        for h in self.transfer_handles:
            for c in h.wait(timeout=per_handle):
                c = c if c.is_graph_completed() else self._join_op_reports(c)
                if c is not None:
                    self._on_completed(c)

    def _join_op_reports(self, c: CompletedOp) -> Optional[CompletedOp]:
        """Several transfer handles (the nodes of a group that spans nodes) each run every op on their own slice
        of the blocks. An op counts once ALL of them reported it: only then may its callback publish the blocks.
        Success and per-block results are combined with AND; a handle that reports no per-block list, or one of
        another length, where another handle reported one fails every block (reference scenarios:
        tests/test_kvtask_lifecycle.py multi-handle block results)."""
        key = (c.graph_id, c.op_id)
        with self._lock:
            rec = self._op_reports.get(key)
            if rec is None:
                rec = self._op_reports[key] = [0, True, [], 0.0, 0]
            rec[0] += 1
            rec[1] = rec[1] and bool(c.success)
            rec[2].append(c.block_results)
            rec[3] = max(rec[3], float(c.gpu_ms))
            rec[4] += int(c.num_bytes)
            if rec[0] < len(self.transfer_handles):
                return None
            del self._op_reports[key]
        lists = rec[2]
        results = None
        if any(r is not None for r in lists):
            n = max(len(r) for r in lists if r is not None)
            if any(r is None or len(r) != n for r in lists):
                results = (False,) * n
            else:
                results = tuple(all(col) for col in zip(*lists))
        return CompletedOp(c.graph_id, c.op_id, rec[1], block_results=results, gpu_ms=rec[3], num_bytes=rec[4])

    def pump(self, timeout: float) -> None:
        """Blocks up to ``timeout`` seconds for the next completion of the data plane and applies what arrived.
        A server calls this between requests while clients wait for tasks."""
        self._update_tasks(timeout=timeout)

    def completion_fds(self) -> Optional[List[int]]:
        """One pollable descriptor per transfer handle, or None when some handle has none (a data plane in
        another process, the Python scheduler): the caller then has to poll on a timer."""
        fds = []
        for h in self.transfer_handles:
            fd = h.completion_fd() if hasattr(h, "completion_fd") else -1
            if fd < 0:
                return None
            fds.append(fd)
        return fds

    def _member_tasks(self, task: KVTask) -> List[KVTask]:
        if not task.children:
            return [task]
        return [self.tasks[c] for c in task.children if c in self.tasks]

    def _on_completed(self, c: CompletedOp) -> None:
        with self._lock:
            tid = self.graph_to_task.get(c.graph_id)
            if tid is None:
                return
            task = self.tasks.get(tid)
            if task is None:
                return
            if c.is_graph_completed():
                task.any_failed = task.any_failed or not c.success
                task.handles_pending -= 1
                if task.handles_pending > 0:
                    return                       # every handle must report before the task ends
                self.graph_to_task.pop(c.graph_id, None)
                if self._op_reports:                     # ops of a failed graph that not every handle reported
                    for key in [k for k in self._op_reports if k[0] == c.graph_id]:
                        del self._op_reports[key]
                self._finish_task(task, success=not task.any_failed)
                return
            if not c.success:
                task.any_failed = True
                return
            # per-op callbacks (mark index nodes ready) run once per op, after every handle reported it
            members = self._member_tasks(task)
            if task.children:
                for m in members:
                    for old, new in task.op_remap.items():
                        if new == c.op_id and old in m.op_callback_dict:
                            self.cache_engine.run_op_callback(m.op_callback_dict.pop(old), c)
            else:
                cb = task.op_callback_dict.pop(c.op_id, None)
                if cb is not None:
                    self.cache_engine.run_op_callback(cb, c)
            if c.op_id == task.task_end_op_id:
                task.task_end_op_finished = True
                for m in members:
                    m.task_end_op_finished = True

    def _finish_task(self, task: KVTask, success: bool) -> None:
        for m in self._member_tasks(task):
            if m.is_completed():
                continue
            m.status = TaskStatus.COMPLETED if success else TaskStatus.FAILED
            m.task_end_op_finished = True
            if m.plan_handle is not None:
                (m.plan_handle.complete if success else m.plan_handle.abort)()
                part = getattr(getattr(m.plan_handle, "plan", None), "partial_blocks", None)
                if success and part is not None and isinstance(m.return_mask, np.ndarray) and m.return_mask.any():
                    # only the longest prefix that really arrived is reported (flexkv/kvtask.py:615-698)
                    first = int(np.flatnonzero(m.return_mask)[0])
                    m.return_mask = m.return_mask.copy()
                    m.return_mask[first + part * self.cache_config.tokens_per_block:] = False
            if not success and m.task_type == TaskType.GET and m.slot_mapping is not None:
                m.failed_gpu_blocks = slot_mapping_to_block_ids(np.asarray(m.slot_mapping, dtype=np.int64),
                                                                self.cache_config.tokens_per_block)
            log_op(m.task_type.value, "finish", "ok" if success else "failed", task_id=m.task_id)
            m.shed_heavy_resources()
        if task.children:
            task.status = TaskStatus.COMPLETED if success else TaskStatus.FAILED
            task.task_end_op_finished = True
            task.shed_heavy_resources()

    def _response(self, task: KVTask) -> KVResponse:
        if task.is_completed():
            return KVResponse(_STATUS_MAP[task.status], task.task_id, task.return_mask)
        # end op finished, rest of the graph still running
        return KVResponse(KVResponseStatus.SUCCESS, task.task_id, task.return_mask)

    def _done_for_wait(self, task: KVTask, completely: bool) -> bool:
        if task.is_completed():
            return True
        return (not completely) and task.task_end_op_finished and not task.any_failed

    def wait(self, task_ids: Union[int, List[int]], timeout: float = 20.0, completely: bool = False
             ) -> Dict[int, KVResponse]:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        self.tracer.trace_wait(task_ids, timeout, completely)
        deadline = time.monotonic() + timeout
        out: Dict[int, KVResponse] = {}
        for tid in task_ids:
            task = self.tasks.get(tid)
            if task is None:
                out[tid] = KVResponse(KVResponseStatus.NOTFOUND, tid, None)
                continue
            if task.status in (TaskStatus.UNREADY, TaskStatus.READY) and task.parent < 0:
                out[tid] = KVResponse(KVResponseStatus.UNREADY, tid, None)
                continue
            while not self._done_for_wait(task, completely):
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                self._update_tasks(timeout=min(left, 0.05))
            if self._done_for_wait(task, completely):
                out[tid] = self._response(task)
                if task.is_completed():
                    self._release(task)
            else:
                out[tid] = KVResponse(KVResponseStatus.TIMEOUT, tid, None)
        return out

    def wait_would_return_now(self, task_ids: List[int], completely: bool = False) -> bool:
        """True when ``wait(task_ids, ...)`` has nothing left to wait for (every task is finished, unknown or not
        launched). Consumes nothing: a server parks a blocking wait until this holds and serves other clients
        meanwhile."""
        self._update_tasks(timeout=0)
        for tid in task_ids:
            task = self.tasks.get(tid)
            if task is None or (task.status in (TaskStatus.UNREADY, TaskStatus.READY) and task.parent < 0):
                continue
            if not self._done_for_wait(task, completely):
                return False
        return True

    def try_wait(self, task_ids: Union[int, List[int]]) -> Dict[int, KVResponse]:
        if isinstance(task_ids, int):
            task_ids = [task_ids]
        self._update_tasks(timeout=0)
        out: Dict[int, KVResponse] = {}
        for tid in task_ids:
            task = self.tasks.get(tid)
            if task is None:
                out[tid] = KVResponse(KVResponseStatus.NOTFOUND, tid, None)
            elif self._done_for_wait(task, completely=False):
                out[tid] = self._response(task)
                if task.is_completed():
                    self._release(task)
        return out

    def _release(self, task: KVTask) -> None:
        with self._lock:
            for c in task.children:
                self.tasks.pop(c, None)
            self.tasks.pop(task.task_id, None)

    def get_failed_gpu_blocks(self, task_id: int) -> Optional[np.ndarray]:
        t = self.tasks.get(task_id)
        return None if t is None else t.failed_gpu_blocks

    # ---- GPU prefix sharing --------------------------------------------------------
    def publish_gpu_blocks(self, token_ids: np.ndarray, slot_mapping: np.ndarray, dp_id: int = 0,
                           namespace: Optional[List[str]] = None) -> int:
        ids = slot_mapping_to_block_ids(np.asarray(slot_mapping, dtype=np.int64), self.cache_config.tokens_per_block)
        return self.cache_engine.publish_gpu_blocks(dp_id, token_ids, ids, namespace)

    def withdraw_gpu_blocks(self, gpu_block_ids: np.ndarray, dp_id: int = 0) -> List[int]:
        return self.cache_engine.withdraw_gpu_blocks(dp_id, gpu_block_ids)

    # ---- maintenance ----------------------------------------------------------
    def _clear_cpu_cache(self) -> None:
        self.cache_engine.cpu_cache_engine.reset()

    def reset_cache(self) -> None:
        """Invalidates every tier. Unlaunched tasks are cancelled; transfers in
        flight finish, but their completion callbacks no longer touch the new
        (empty) index (flexkv/kvtask.py:1446-1488)."""
        self._update_tasks(timeout=0)
        with self._lock:
            for task in list(self.tasks.values()):
                if task.is_completed():
                    continue
                if task.status in (TaskStatus.UNREADY, TaskStatus.READY) and task.parent < 0:
                    task.status = TaskStatus.CANCELLED
                    self.graph_to_task.pop(task.graph.graph_id, None)
                # neuter: nodes named by the plan belong to the index that is being dropped
                task.op_callback_dict = {}
                if task.plan_handle is not None:
                    task.plan_handle._once()   # noqa: SLF001 - marks the handle spent without running it
            self._epoch += 1
            self.cache_engine.reset()
        self.tracer.trace_reset()
