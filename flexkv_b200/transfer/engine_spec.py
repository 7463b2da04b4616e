"""Data-plane runtime, Python specification: a scheduler thread that walks transfer graphs
and hands ready ops to per-type workers. The production engine (``engine.py``) keeps the graph
state in the native ``GraphScheduler`` and dispatches without a scheduler thread; this module is
its executable specification (same worker protocol, same completion records), selected with
``FLEXKV_NATIVE_SCHEDULER=0`` and used by the differential tests.

The reference runs one *process* per worker type behind two pipe hops
(flexkv/transfer/transfer_engine.py:443-760,1115-1286; flexkv/transfer/worker.py).
Here workers are threads of the serving process: the heavy lifting happens in
native code that releases the GIL (kernel launches joined on CUDA events,
io_uring submission), so an op costs one queue hand-off instead of pickling
through pipes, and block ids reach the GPU through a mapped pinned ring with no
shared-memory slot pool. Failure semantics are the reference's: a failed op
stops further dispatch of its graph, in-flight ops drain, and the graph is
reported once as failed (flexkv/transfer/transfer_engine.py:1320-1378).
"""
from __future__ import annotations

import queue
import threading
from typing import Dict, List, Optional, Tuple


from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from ..common.debug import flexkv_logger
from ..common.transfer import (CompletedOp, LayerwiseTransferOp, TransferOp, TransferOpGraph, TransferType,
                               WorkerKey)
from .trace import TransferTrace
from .workers import OpOutcome, TransferWorker, build_workers


_GPU_TYPES = (TransferType.H2D, TransferType.D2H, TransferType.LAYERWISE, TransferType.PEERD2D, TransferType.DISK2D,
              TransferType.D2DISK)


class TransferEngineSpec:
    def __init__(self, storage, model_config: ModelConfig, cache_config: CacheConfig,
                 workers: Optional[Dict[Tuple[WorkerKey, TransferType], TransferWorker]] = None) -> None:
        self.storage = storage
        self.model_config = model_config
        self.cache_config = cache_config
        self._events: "queue.Queue[Tuple[str, Any, Any]]" = queue.Queue()
        self._completed: "queue.Queue[CompletedOp]" = queue.Queue()
        self._graphs: Dict[int, TransferOpGraph] = {}
        self._inflight: Dict[int, int] = {}
        self._workers = workers
        self._thread: Optional[threading.Thread] = None
        self._ready = threading.Event()
        self._stopping = False
        self._trace = TransferTrace(enabled=GLOBAL_CONFIG_FROM_ENV.enable_transfer_trace)
        self._metrics = None
        # sleep/wake of the engine's GPU memory: ops that touch a suspended client's GPU are parked
        self._suspended: set = set()
        self._parked: List[Tuple[TransferOpGraph, TransferOp]] = []
        self._gpu_inflight: Dict[WorkerKey, int] = {}
        self._drain_waiters: List[Tuple[set, threading.Event]] = []
        self._pp_acc: Dict[int, list] = {}      # op id -> [all ok, bytes, max ms, first error, -] over pipeline stages
        self.stats = dict(ops=0, failed_ops=0, graphs=0, failed_graphs=0)
        self.stats_by_type: Dict[str, List[float]] = {}     # type -> [ops, blocks, bytes, kernel or IO ms]

    # ---- lifecycle ------------------------------------------------------------
    def start(self) -> None:
        if self._workers is None:
            self._workers = build_workers(self.storage, self.model_config, self.cache_config)
        for w in set(self._workers.values()):
            w.start(self._on_worker_done)
        self._thread = threading.Thread(target=self._loop, name="flexkv-scheduler", daemon=True)
        self._thread.start()
        self._ready.set()

    def is_ready(self) -> bool:
        return self._ready.is_set()

    def set_metrics_collector(self, collector) -> None:
        self._metrics = collector

    def shutdown(self) -> None:
        if self._thread is None:
            return
        self._stopping = True
        self._events.put(("stop", None, None))
        self._thread.join(timeout=30)
        self._thread = None
        for w in set((self._workers or {}).values()):
            w.stop()
        self._ready.clear()

    def worker_for(self, key: WorkerKey, tt: TransferType) -> Optional[TransferWorker]:
        return (self._workers or {}).get((key, tt))

    # ---- submission / completion ----------------------------------------------
    def submit(self, graph: TransferOpGraph) -> None:
        self._events.put(("submit", graph, None))

    def submit_batch(self, graphs: List[TransferOpGraph]) -> None:
        for g in graphs:
            self._events.put(("submit", g, None))

    def wait(self, timeout: Optional[float] = None) -> List[CompletedOp]:
        """Completed ops so far; blocks up to ``timeout`` seconds for the first one."""
        out: List[CompletedOp] = []
        try:
            if timeout is None or timeout > 0:
                out.append(self._completed.get(timeout=timeout))
            while True:
                out.append(self._completed.get_nowait())
        except queue.Empty:
            pass
        return out

    get_completed_graphs_and_ops = wait

    # ---- scheduler ------------------------------------------------------------
    def _on_worker_done(self, op: TransferOp, outcome: OpOutcome) -> None:
        self._events.put(("done", op, outcome))

    def _loop(self) -> None:
        while True:
            kind, a, b = self._events.get()
            if kind == "stop":
                break
            try:
                if kind == "submit":
                    self._on_submit(a)
                elif kind == "done":
                    self._on_done(a, b)
                elif kind == "suspend":
                    self._on_suspend(a, b)
                elif kind == "resume":
                    self._on_resume(a, b)
            except Exception:  # noqa: BLE001  - the scheduler must survive a bad graph
                flexkv_logger.exception("transfer scheduler error")

    def _on_submit(self, graph: TransferOpGraph) -> None:
        self._graphs[graph.graph_id] = graph
        self._inflight[graph.graph_id] = 0
        self.stats["graphs"] += 1
        if graph.num_ops == 0:
            self._finish_graph(graph)
            return
        self._dispatch(graph)

    def _dispatch(self, graph: TransferOpGraph) -> None:
        progress = not graph.failed        # a failed graph gets no new ops; in-flight ones drain
        while progress:
            progress = False
            for op in graph.take_ready_ops():
                if op.transfer_type == TransferType.VIRTUAL or (op.valid_block_num == 0 and
                                                                not isinstance(op, LayerwiseTransferOp)):
                    graph.mark_completed(op.op_id, True)
                    self._completed.put(CompletedOp(graph.graph_id, op.op_id, True))
                    progress = True
                    continue
                key = WorkerKey(op.dp_client_id, 0)
                if key in self._suspended and op.transfer_type in _GPU_TYPES:
                    self._parked.append((graph, op))       # runs after resume_gpu_mappings
                    continue
                w = self._workers.get((key, "SWA" if op.is_swa else op.transfer_type))
                if w is None and not op.is_swa and op.transfer_type not in (TransferType.H2D, TransferType.D2H, TransferType.LAYERWISE,
                                                          TransferType.PEERD2D, TransferType.DISK2D,
                                                          TransferType.D2DISK):
                    # tier-to-tier workers (SSD, remote) are shared by every data-parallel client
                    w = self._workers.get((WorkerKey(0, 0), op.transfer_type))
                if w is None:
                    flexkv_logger.error("no worker for %s (dp client %d)", op.transfer_type.value, op.dp_client_id)
                    graph.mark_completed(op.op_id, False)
                    self._completed.put(CompletedOp(graph.graph_id, op.op_id, False))
                    continue
                self._inflight[graph.graph_id] += 1
                if op.transfer_type in _GPU_TYPES:
                    self._gpu_inflight[key] = self._gpu_inflight.get(key, 0) + 1
                self._trace.on_submit(op)
                # pipeline stages served by this manager each hold their own layers of the same blocks: the op
                # goes to every stage's worker and counts as done when the last of them reports
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
                    self._pp_acc[op.op_id] = [True, 0, 0.0, "", None]
                for sw in siblings:
                    sw.submit(op)
        if graph.all_transfer_ops_completed() or (graph.failed and self._inflight[graph.graph_id] == 0):
            self._finish_graph(graph)

    # ---- sleep / wake -----------------------------------------------------------
    def suspend_gpu_mappings(self, dp_client_id: Optional[int] = None, timeout: float = 60.0) -> bool:
        """Stops touching the GPU memory of one data-parallel client (all when None): ops that
        need it are parked, and the call returns once none is in flight, so the engine may
        release or remap that memory (vLLM sleep mode; flexkv/transfer/transfer_engine.py:1661-1716).
        The host, SSD and remote tiers keep working."""
        keys = {k for k in (self.storage.gpu_regs if self.storage is not None else {})
                if dp_client_id is None or k.dp_client_id == dp_client_id}
        ev = threading.Event()
        self._events.put(("suspend", keys, ev))
        return ev.wait(timeout)

    def resume_gpu_mappings(self, dp_client_id: Optional[int] = None, new_registrations=None) -> None:
        """``new_registrations``: GpuRegistration objects of the re-created tensors (same geometry,
        new addresses); omitted when the memory came back at the old addresses."""
        keys = {k for k in (self.storage.gpu_regs if self.storage is not None else {})
                if dp_client_id is None or k.dp_client_id == dp_client_id}
        done = threading.Event()
        self._events.put(("resume", (keys, list(new_registrations or [])), done))
        done.wait(60.0)

    def _on_suspend(self, keys: set, ev: threading.Event) -> None:
        self._suspended |= keys
        if all(self._gpu_inflight.get(k, 0) == 0 for k in keys):
            ev.set()
        else:
            self._drain_waiters.append((keys, ev))

    def _on_resume(self, arg, done: threading.Event) -> None:
        keys, regs = arg
        try:
            for reg in regs:
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
            touched = []
            for graph, op in parked:
                if WorkerKey(op.dp_client_id, 0) in self._suspended:
                    self._parked.append((graph, op))
                    continue
                graph.requeue(op.op_id)
                if graph not in touched:
                    touched.append(graph)
            for g in touched:
                self._dispatch(g)
        finally:
            done.set()

    def _on_done(self, op: TransferOp, outcome: OpOutcome) -> None:
        acc = self._pp_acc.get(op.op_id)
        if acc is not None:
            # one report per pipeline stage: fold, and go on only with the last one
            acc[0] = acc[0] and outcome.success
            acc[1] += outcome.num_bytes
            acc[2] = max(acc[2], outcome.gpu_ms)
            acc[3] = acc[3] or outcome.error
            op.pending_count -= 1
            if op.pending_count > 0:
                return
            del self._pp_acc[op.op_id]
            outcome = OpOutcome(acc[0], gpu_ms=acc[2], num_bytes=acc[1], error=acc[3])
        if op.transfer_type in _GPU_TYPES:
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
        graph = self._graphs.get(op.graph_id)
        if graph is None:
            return
        self._inflight[graph.graph_id] -= 1
        self.stats["ops"] += 1
        if not outcome.success:
            self.stats["failed_ops"] += 1
        op.block_results = outcome.block_results
        acc = self.stats_by_type.setdefault(op.transfer_type.value, [0, 0, 0, 0.0])
        acc[0] += 1
        acc[1] += op.valid_block_num
        acc[2] += outcome.num_bytes
        acc[3] += outcome.gpu_ms
        self._trace.on_done(op, outcome)
        if self._metrics is not None:
            self._metrics.record_transfer(op.transfer_type.value, op.valid_block_num, outcome.num_bytes,
                                          outcome.success)
        graph.mark_completed(op.op_id, outcome.success)
        self._completed.put(CompletedOp(graph.graph_id, op.op_id, outcome.success,
                                        block_results=outcome.block_results, gpu_ms=outcome.gpu_ms,
                                        num_bytes=outcome.num_bytes))
        self._dispatch(graph)

    def _finish_graph(self, graph: TransferOpGraph) -> None:
        if graph.graph_id not in self._graphs:
            return
        del self._graphs[graph.graph_id]
        del self._inflight[graph.graph_id]
        if graph.failed:
            self.stats["failed_graphs"] += 1
        self._completed.put(CompletedOp.graph_done(graph.graph_id, success=not graph.failed))
