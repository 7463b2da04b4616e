"""Data-plane runtime: transfer graphs scheduled by the native ``GraphScheduler``, ops executed by
per-type workers.

The graph state (ready set, dependency release, fan-out joins over pipeline stages, failure drain,
completion queue) lives in C++ (``csrc/graph_scheduler.{h,cpp}``). There is no scheduler thread: a
submission dispatches the graph's root ops from the caller's thread, and the worker thread that
finishes an op releases and dispatches its successors itself, so an op costs one queue hand-off to
its worker and one GIL-free wait on the native completion queue. The reference runs a scheduler
thread on a selector loop between two pipe hops and one *process* per worker type
(flexkv/transfer/transfer_engine.py:443-760,1115-1286; flexkv/transfer/worker.py). Failure
semantics are the reference's: a failed op stops further dispatch of its graph, in-flight ops drain,
and the graph is reported once as failed (flexkv/transfer/transfer_engine.py:1320-1378).
``engine_spec.py`` is the Python specification of the same behaviour.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Tuple

from .. import _native
from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from ..common.debug import flexkv_logger
from ..common.transfer import (CompletedOp, LayerwiseTransferOp, TransferOp, TransferOpGraph, TransferOpStatus,
                               TransferType, WorkerKey)
from .trace import TransferTrace
from .workers import OpOutcome, TransferWorker, build_workers

_GPU_TYPES = (TransferType.H2D, TransferType.D2H, TransferType.LAYERWISE, TransferType.PEERD2D, TransferType.DISK2D,
              TransferType.D2DISK)


class TransferEngine:
    def __init__(self, storage, model_config: ModelConfig, cache_config: CacheConfig,
                 workers: Optional[Dict[Tuple[WorkerKey, TransferType], TransferWorker]] = None) -> None:
        self.storage = storage
        self.model_config = model_config
        self.cache_config = cache_config
        self._sched = _native.C.GraphScheduler()
        self._lock = threading.RLock()          # dispatch state below; the graph state has its own native lock
        self._graphs: Dict[int, TransferOpGraph] = {}
        self._block_results: Dict[Tuple[int, int], tuple] = {}
        self._workers = workers
        self._started = False
        self._ready = threading.Event()
        self._trace = TransferTrace(enabled=GLOBAL_CONFIG_FROM_ENV.enable_transfer_trace)
        self._metrics = None
        # sleep/wake of the engine's GPU memory: ops that touch a suspended client's GPU are parked
        self._suspended: set = set()
        self._parked: List[Tuple[TransferOpGraph, TransferOp]] = []
        self._gpu_inflight: Dict[WorkerKey, int] = {}
        self._drain_waiters: List[Tuple[set, threading.Event]] = []
        self.stats_by_type: Dict[str, List[float]] = {}     # type -> [ops, blocks, bytes, kernel or IO ms]

    @property
    def stats(self) -> Dict[str, int]:
        return dict(self._sched.stats())

    # ---- lifecycle ------------------------------------------------------------
    def start(self) -> None:
        if self._workers is None:
            self._workers = build_workers(self.storage, self.model_config, self.cache_config)
        for w in set(self._workers.values()):
            w.start(self._on_worker_done)
        self._started = True
        self._ready.set()

    def is_ready(self) -> bool:
        return self._ready.is_set()

    def set_metrics_collector(self, collector) -> None:
        self._metrics = collector

    def shutdown(self) -> None:
        if not self._started:
            return
        self._started = False
        for w in set((self._workers or {}).values()):
            w.stop()
        self._ready.clear()

    def worker_for(self, key: WorkerKey, tt: TransferType) -> Optional[TransferWorker]:
        return (self._workers or {}).get((key, tt))

    # ---- submission / completion ----------------------------------------------
    def submit(self, graph: TransferOpGraph) -> None:
        ops = graph.ops()
        ids = [op.op_id for op in ops]
        instant = _native.C.SCHED_OP_INSTANT
        flags = [instant if (op.transfer_type == TransferType.VIRTUAL or
                             (op.valid_block_num == 0 and not isinstance(op, LayerwiseTransferOp))) else 0
                 for op in ops]
        edges = [(op.op_id, p) for op in ops for p in op.predecessors]
        with self._lock:
            self._graphs[graph.graph_id] = graph
            try:
                ready = self._sched.submit(graph.graph_id, ids, flags, edges)
            except Exception:  # noqa: BLE001 - a malformed graph must not take the data plane down
                flexkv_logger.exception("transfer graph %d rejected", graph.graph_id)
                del self._graphs[graph.graph_id]
                raise
            for op, f in zip(ops, flags):
                if f:
                    op.status = TransferOpStatus.COMPLETED
            if not self._sched.has_graph(graph.graph_id):      # nothing but instant ops
                self._graphs.pop(graph.graph_id, None)
            for oid in ready:
                self._dispatch_op(graph, graph.get_op(oid))

    def submit_batch(self, graphs: List[TransferOpGraph]) -> None:
        for g in graphs:
            self.submit(g)

    def wait(self, timeout: Optional[float] = None) -> List[CompletedOp]:
        """Completed ops so far; blocks up to ``timeout`` seconds for the first one."""
        recs = self._sched.wait(-1.0 if timeout is None else float(timeout))
        out: List[CompletedOp] = []
        for gid, oid, ok, ms, nbytes in recs:
            if oid < 0:
                out.append(CompletedOp.graph_done(gid, success=ok))
            else:
                br = self._block_results.pop((gid, oid), None) if self._block_results else None
                out.append(CompletedOp(gid, oid, ok, block_results=br, gpu_ms=ms, num_bytes=nbytes))
        return out

    get_completed_graphs_and_ops = wait

    def completion_fd(self) -> int:
        """Descriptor that is readable while ``wait(0)`` would return records (the native scheduler's eventfd)."""
        return int(self._sched.completion_fd())

    # ---- dispatch ---------------------------------------------------------------
    def _dispatch_op(self, graph: TransferOpGraph, op: TransferOp) -> None:
        """Hands one released op to its worker(s). Called with the lock held."""
        op.status = TransferOpStatus.RUNNING
        key = WorkerKey(op.dp_client_id, 0)
        if key in self._suspended and op.transfer_type in _GPU_TYPES:
            self._sched.requeue(graph.graph_id, op.op_id)
            op.status = TransferOpStatus.PENDING
            self._parked.append((graph, op))       # runs after resume_gpu_mappings
            return
        w = self._workers.get((key, "SWA" if op.is_swa else op.transfer_type))
        if w is None and not op.is_swa and op.transfer_type not in _GPU_TYPES:
            # tier-to-tier workers (SSD, remote) are shared by every data-parallel client
            w = self._workers.get((WorkerKey(0, 0), op.transfer_type))
        if w is None:
            flexkv_logger.error("no worker for %s (dp client %d)", op.transfer_type.value, op.dp_client_id)
            self._finish_op(op, OpOutcome(False, error="no worker"), count_gpu=False)
            return
        if op.transfer_type in _GPU_TYPES:
            self._gpu_inflight[key] = self._gpu_inflight.get(key, 0) + 1
        self._trace.on_submit(op)
        # pipeline stages served by this manager each hold their own layers of the same blocks: the op goes to
        # every stage's worker and counts as done when the last of them reports
        # (flexkv/transfer/transfer_engine.py:1434-1492,1562-1613)
        siblings = [w]
        if op.transfer_type in (TransferType.H2D, TransferType.D2H) and not op.is_swa \
                and self.model_config.local_pp_stages > 1:
            for r in range(1, self.model_config.local_pp_stages):
                sw = self._workers.get((WorkerKey(op.dp_client_id, r), op.transfer_type))
                if sw is not None:
                    siblings.append(sw)
        op.pending_count = len(siblings)
        if len(siblings) > 1:
            self._sched.set_fanout(graph.graph_id, op.op_id, len(siblings))
        for sw in siblings:
            sw.submit(op)

    def _on_worker_done(self, op: TransferOp, outcome: OpOutcome) -> None:
        """Runs on the worker's thread."""
        try:
            with self._lock:
                self._finish_op(op, outcome, count_gpu=True)
        except Exception:  # noqa: BLE001  - a worker thread must survive a bad completion
            flexkv_logger.exception("transfer scheduler error")

    def _finish_op(self, op: TransferOp, outcome: OpOutcome, count_gpu: bool) -> None:
        if outcome.block_results is not None:
            self._block_results[(op.graph_id, op.op_id)] = outcome.block_results
            op.block_results = outcome.block_results
        accepted, finished, ok, ms, nbytes, g_done, g_failed, ready = self._sched.op_done(
            op.graph_id, op.op_id, bool(outcome.success), float(outcome.gpu_ms), int(outcome.num_bytes))
        if not accepted:
            self._block_results.pop((op.graph_id, op.op_id), None)
            return
        if not finished:
            op.pending_count -= 1               # other pipeline stages still hold the op
            return
        if count_gpu and op.transfer_type in _GPU_TYPES:
            key = WorkerKey(op.dp_client_id, 0)
            self._gpu_inflight[key] = max(0, self._gpu_inflight.get(key, 0) - 1)
            if self._drain_waiters:
                still = []
                for keys, ev in self._drain_waiters:
                    if all(self._gpu_inflight.get(k, 0) == 0 for k in keys):
                        ev.set()
                    else:
                        still.append((keys, ev))
                self._drain_waiters = still
        op.status = TransferOpStatus.COMPLETED if ok else TransferOpStatus.FAILED
        acc = self.stats_by_type.setdefault(op.transfer_type.value, [0, 0, 0, 0.0])
        acc[0] += 1
        acc[1] += op.valid_block_num
        acc[2] += nbytes
        acc[3] += ms
        self._trace.on_done(op, OpOutcome(ok, gpu_ms=ms, num_bytes=nbytes, error=outcome.error))
        if self._metrics is not None:
            self._metrics.record_transfer(op.transfer_type.value, op.valid_block_num, nbytes, ok)
        graph = self._graphs.get(op.graph_id)
        if graph is None:
            return
        if g_failed:
            graph.failed = True
        if g_done:
            del self._graphs[op.graph_id]
            return
        for oid in ready:
            self._dispatch_op(graph, graph.get_op(oid))

    # ---- sleep / wake -----------------------------------------------------------
    def _keys_of(self, dp_client_id: Optional[int]) -> set:
        return {k for k in (self.storage.gpu_regs if self.storage is not None else {})
                if dp_client_id is None or k.dp_client_id == dp_client_id}

    def suspend_gpu_mappings(self, dp_client_id: Optional[int] = None, timeout: float = 60.0) -> bool:
        """Stops touching the GPU memory of one data-parallel client (all when None): ops that
        need it are parked, and the call returns once none is in flight, so the engine may
        release or remap that memory (vLLM sleep mode; flexkv/transfer/transfer_engine.py:1661-1716).
        The host, SSD and remote tiers keep working."""
        keys = self._keys_of(dp_client_id)
        ev = threading.Event()
        with self._lock:
            self._suspended |= keys
            if all(self._gpu_inflight.get(k, 0) == 0 for k in keys):
                ev.set()
            else:
                self._drain_waiters.append((keys, ev))
        return ev.wait(timeout)

    def resume_gpu_mappings(self, dp_client_id: Optional[int] = None, new_registrations=None) -> None:
        """``new_registrations``: GpuRegistration objects of the re-created tensors (same geometry,
        new addresses); omitted when the memory came back at the old addresses."""
        keys = self._keys_of(dp_client_id)
        with self._lock:
            for reg in list(new_registrations or []):
                key = WorkerKey(reg.dp_client_id, reg.pp_rank)
                gid = int(getattr(reg, "group_id", 0) or 0)
                by_group = self.storage.gpu_group_regs.get(key, {}).get(reg.tp_rank)
                old = by_group.get(gid) if by_group else self.storage.gpu_regs.get(key, {}).get(reg.tp_rank)
                if old is None:
                    raise ValueError(f"resume: no registration for {key} rank {reg.tp_rank}")
                if (old.chunk_bytes, old.num_layers, old.kv_dim, len(old.ptrs)) != \
                        (reg.chunk_bytes, reg.num_layers, reg.kv_dim, len(reg.ptrs)):
                    raise ValueError("resume: the re-registered tensors have a different geometry")
                old.ptrs = list(reg.ptrs)
                old.num_blocks = reg.num_blocks
                old.keepalive = reg.keepalive
                rank_index = sorted(self.storage.gpu_regs[key]).index(reg.tp_rank)
                for (k, _), w in self._workers.items():
                    if k == key and hasattr(w, "update_gpu_ptrs"):
                        if by_group:      # per-group tensors: only the layerwise worker keeps native copies
                            w.update_gpu_ptrs(rank_index, [int(p) for p in reg.ptrs], gid)
                        else:
                            w.update_gpu_ptrs(rank_index, [int(p) for p in reg.ptrs])
                    if hasattr(w, "update_gpu_ptrs_for") and reg.tp_rank == 0 and key.dp_client_id in w.rank_of:
                        w.update_gpu_ptrs_for(key.dp_client_id, [int(p) for p in reg.ptrs])
            self._suspended -= keys
            parked, self._parked = self._parked, []
            touched: List[TransferOpGraph] = []
            for graph, _ in parked:
                if graph not in touched:
                    touched.append(graph)
            # every parked op is handed out again; one whose client is still asleep parks itself again
            for g in touched:
                for oid in self._sched.take_ready(g.graph_id):
                    self._dispatch_op(g, g.get_op(oid))
                if not self._sched.has_graph(g.graph_id):
                    self._graphs.pop(g.graph_id, None)
