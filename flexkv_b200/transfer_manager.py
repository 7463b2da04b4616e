"""Owner of the data plane: storage tiers, GPU registrations and the transfer
engine, behind the handle interface the task layer uses
(``start / is_ready / submit_batch / wait / shutdown``).

The reference spawns this as a separate process and talks to it over pipes
(flexkv/transfer_manager.py:38-527,970-1272); here it lives in the serving
process and initialises on a background thread: GPU registrations may arrive
in-process (``register_gpu``) or from engine worker processes over a ZMQ
PULL socket carrying exported tensor handles (flexkv/transfer_manager.py:77-83,
317-357). Graphs submitted before initialisation finished are queued.
"""
from __future__ import annotations

import os
import threading
import time
from typing import List, Optional

from .common.config import CacheConfig, ModelConfig
from .common.debug import flexkv_logger
from .common.transfer import CompletedOp, TransferOpGraph
from .storage.gpu_layout import GpuRegistration
from .storage.storage_engine import StorageEngine
from .common.config import GLOBAL_CONFIG_FROM_ENV
from .transfer.engine import TransferEngine
from .transfer.engine_spec import TransferEngineSpec


class TransferManager:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, gpu_register_port: Optional[str] = None,
                 require_gpu: bool = True, numa_node: int = -1) -> None:
        self.model_config = model_config
        self.cache_config = cache_config
        self.gpu_register_port = gpu_register_port
        self.require_gpu = require_gpu
        self.numa_node = numa_node
        self.storage: Optional[StorageEngine] = None
        self.engine: Optional[TransferEngine] = None
        self._pending_regs: List[GpuRegistration] = []
        self._pending_swa: List[GpuRegistration] = []
        self._reg_cv = threading.Condition()
        self._ready = threading.Event()
        self._init_error: Optional[BaseException] = None
        self._init_thread: Optional[threading.Thread] = None
        self._early: List[TransferOpGraph] = []
        self._early_lock = threading.Lock()
        self._listener = None
        self._metrics = None
        self._stop = False
        # graphs that arrived with their GPU side unbound, and page lists that arrived before their graph
        self._bind_lock = threading.Lock()
        self._await_pages: dict = {}        # task id -> [graphs]
        self._early_pages: dict = {}        # task id -> slot mapping

    # ---- registration -----------------------------------------------------------
    def register_gpu(self, reg: GpuRegistration) -> None:
        if getattr(reg, "is_swa", False):
            self.register_swa(reg)
            return
        # a caller written against the reference names its rank by ``intra_client_id`` = pp_rank * (tp x cp ranks)
        # + rank inside the stage (flexkv/common/config.py:511-516); the rank inside the stage is what is kept here
        width = int(getattr(self.model_config, "effective_tp_size", 0) or 0)
        if width > 0 and reg.pp_rank > 0 and reg.tp_rank >= width and 0 <= reg.tp_rank - reg.pp_rank * width < width:
            reg.tp_rank -= reg.pp_rank * width
        with self._reg_cv:
            self._pending_regs.append(reg)
            self._reg_cv.notify_all()

    def register_swa(self, reg: GpuRegistration) -> None:
        """Window pages of one rank; must arrive before start() completes initialisation."""
        with self._reg_cv:
            self._pending_swa.append(reg)
            self._reg_cv.notify_all()

    def _expected_swa_registrations(self) -> int:
        """Window registrations that start-up waits for: every rank, every group of the window pool."""
        swa = self.cache_config.swa
        if swa is None or not swa.enabled or not swa.wait_for_registration or not self.require_gpu:
            return 0
        m = self.model_config
        return m.total_clients * m.local_pp_stages * m.effective_tp_size_per_node * (1 + len(swa.sidecar_groups))

    def _adopt_layer_groups(self) -> None:
        """Layer groups discovered by an engine worker (first list wins) when this side was configured with
        none. Block counts stay as the planner knows them; only the block size grows."""
        if self.model_config.layer_groups:
            return
        for r in self._pending_regs:
            groups = getattr(r, "layer_groups", None)
            if groups:
                object.__setattr__(self.model_config, "layer_groups", list(groups))
                flexkv_logger.info("layer groups taken from the GPU registration of rank %d: %s", r.tp_rank,
                                   [(g.num_layers, g.num_kv_heads, g.head_size, g.compress_ratio) for g in groups])
                return

    def _expected_registrations(self) -> int:
        self._adopt_layer_groups()
        m = self.model_config
        groups = len(m.layer_groups) if m.layer_groups else 1      # one registration per rank and layer group
        return m.total_clients * m.local_pp_stages * m.effective_tp_size_per_node * groups if self.require_gpu else 0

    def _registrations_arrived(self) -> int:
        """A registration with multicast addresses stands for every rank of its tensor-parallel group."""
        per_group = self.model_config.effective_tp_size_per_node
        return sum(per_group if getattr(r, "mc_ptrs", None) else 1 for r in self._pending_regs)

    # ---- lifecycle ----------------------------------------------------------------
    def start(self) -> None:
        if self._init_thread is not None:
            return
        if self.gpu_register_port:
            from .server.registration import RegistrationListener
            self._listener = RegistrationListener(self.gpu_register_port, self.register_gpu, self._on_gpu_control,
                                                  lambda req: self.set_slot_mapping(req.task_id, req.slot_mapping))
            self._listener.start()
        self._init_thread = threading.Thread(target=self._init, name="flexkv-tm-init", daemon=True)
        self._init_thread.start()

    def _init(self) -> None:
        try:
            want, want_swa = self._expected_registrations(), self._expected_swa_registrations()
            t0 = time.monotonic()
            warned = False
            with self._reg_cv:
                while (self._registrations_arrived() < want or len(self._pending_swa) < want_swa) and not self._stop:
                    self._reg_cv.wait(timeout=1.0)
                    want = self._expected_registrations()      # a registration may have brought the layer groups
                    if not warned and time.monotonic() - t0 > 60:
                        warned = True
                        flexkv_logger.warning("still waiting for GPU registrations: %d of %d arrived (window pages: "
                                              "%d of %d)", self._registrations_arrived(), want, len(self._pending_swa),
                                              want_swa)
            if self._stop:
                return
            numa = self.numa_node
            if numa < 0 and self._pending_regs and self._pending_regs[0].device_id >= 0:
                from . import _native
                numa = _native.C.gpu_numa_node(self._pending_regs[0].device_id)
            has_gpu = any(r.device_id >= 0 for r in self._pending_regs)
            self.storage = StorageEngine(self.model_config, self.cache_config, cuda_register=has_gpu,
                                         numa_node=numa)
            for r in self._pending_regs:
                self.storage.register_gpu_blocks(r)
            for r in self._pending_swa:
                self.storage.register_swa_blocks(r)
            if self.cache_config.enable_p2p_cpu and self.storage.host is not None:
                # what a peer needs to read this node's host pool
                from .cache.hie_cache_engine import get_node_registry
                reg = get_node_registry(self.cache_config, self.model_config)
                reg.set_node_meta(dict(pool_file=self.storage.host_backing_file,
                                       block_bytes=self.storage.host.block_bytes,
                                       num_blocks=self.storage.host.num_blocks, pid=os.getpid(),
                                       codec=self.storage.host.quant))
            if self.cache_config.enable_p2p_ssd and self.storage.ssd is not None:
                # what a peer needs to read this node's SSD blocks out of their files
                import json
                from .cache.hie_cache_engine import get_node_registry
                reg = get_node_registry(self.cache_config, self.model_config)
                ssd = self.storage.ssd
                reg.set_node_meta(dict(ssd_files=json.dumps(ssd.files), ssd_block_bytes=ssd.block_bytes,
                                       ssd_blocks_per_file=ssd.blocks_per_file, ssd_num_blocks=ssd.num_blocks,
                                       ssd_layout=json.dumps(self.storage.ssd_layout_dict(), sort_keys=True),
                                       codec=self.storage.host.quant))
            if self.cache_config.enable_3rd_remote and self.cache_config.enable_remote and \
                    not self.cache_config.use_mooncake_store_backend and self.storage.host is not None:
                # what a peer needs to read the files this node writes to the shared remote file system
                import json
                from .cache.hie_cache_engine import get_node_registry
                from .external.remote_store import get_backend
                backend = get_backend(self.cache_config, self.storage.host.block_bytes)
                if backend is not None and getattr(backend, "files", None):
                    get_node_registry(self.cache_config, self.model_config).set_node_meta(dict(
                        remote_files=json.dumps(backend.files), remote_block_bytes=backend.block_bytes,
                        remote_num_blocks=backend.num_blocks, codec=self.storage.host.quant))
            # graph state in the native scheduler (default) or the Python specification of it
            engine_cls = TransferEngine if GLOBAL_CONFIG_FROM_ENV.native_scheduler else TransferEngineSpec
            self.engine = engine_cls(self.storage, self.model_config, self.cache_config)
            if self._metrics is not None:
                self.engine.set_metrics_collector(self._metrics)
            self.engine.start()
            with self._early_lock:
                early, self._early = self._early, []
                self._ready.set()
            if early:
                self.engine.submit_batch(early)
        except BaseException as e:  # noqa: BLE001
            self._init_error = e
            flexkv_logger.exception("transfer manager initialisation failed")

    def is_ready(self) -> bool:
        if self._init_error is not None:
            raise RuntimeError(f"transfer manager failed to start: {self._init_error}") from self._init_error
        return self._ready.is_set()

    def set_metrics_collector(self, collector) -> None:
        self._metrics = collector
        if self.engine is not None:
            self.engine.set_metrics_collector(collector)

    def suspend_gpu_mappings(self, dp_client_id: Optional[int] = None, timeout: float = 60.0) -> bool:
        if self.engine is None:
            return True
        return self.engine.suspend_gpu_mappings(dp_client_id, timeout)

    def resume_gpu_mappings(self, dp_client_id: Optional[int] = None, new_registrations=None) -> None:
        if self.engine is not None:
            self.engine.resume_gpu_mappings(dp_client_id, new_registrations)

    def _on_gpu_control(self, req) -> bool:
        """Sleep / wake requests of engine worker processes (their tensors are IPC mappings here)."""
        from .server.registration import registration_from_request
        if req.action == "suspend":
            ok = self.suspend_gpu_mappings(req.dp_client_id, req.timeout)
            if ok and self.storage is not None:
                # drop this process's view of the memory so that the owner can really free it
                for key, ranks in self.storage.gpu_regs.items():
                    if key.dp_client_id != req.dp_client_id:
                        continue
                    by_group = self.storage.gpu_group_regs.get(key, {})
                    every = list(ranks.values()) + [g for per_rank in by_group.values() for g in per_rank.values()]
                    seen = set()
                    for reg in every:
                        for h in (reg.keepalive or []):
                            if hasattr(h, "close") and id(h) not in seen:
                                seen.add(id(h))
                                h.close()
            return ok
        if req.action == "resume":
            reqs = ([req.registration] if req.registration is not None else []) + \
                list(getattr(req, "more_registrations", None) or [])
            regs = [registration_from_request(r) for r in reqs]
            self.resume_gpu_mappings(req.dp_client_id, regs)
            return True
        return False

    def submit(self, graph: TransferOpGraph) -> None:
        self.submit_batch([graph])

    def submit_batch(self, graphs: List[TransferOpGraph]) -> None:
        ready_graphs = []
        for g in graphs:
            tid = getattr(g, "bind_task_id", None)
            if tid is None or g.gpu_bound:
                ready_graphs.append(g)
                continue
            # planned on another node: the GPU side is bound from this node's own page list
            with self._bind_lock:
                pages = self._early_pages.pop(tid, None)
                if pages is None:
                    self._await_pages.setdefault(tid, []).append(g)
                    continue
            self._bind(g, pages)
            ready_graphs.append(g)
        graphs = ready_graphs
        if not graphs:
            return
        with self._early_lock:
            if not self._ready.is_set():
                self._early.extend(graphs)
                return
        self.engine.submit_batch(graphs)

    def _bind(self, graph: TransferOpGraph, slot_mapping) -> None:
        import numpy as np
        T = int(self.cache_config.tokens_per_block)
        sm = np.asarray(slot_mapping, dtype=np.int64)
        graph.set_gpu_blocks(sm[::T] // T)

    def set_slot_mapping(self, task_id: int, slot_mapping) -> None:
        """This node's GPU pages for a task planned elsewhere; releases the graphs that waited for them."""
        with self._bind_lock:
            held = self._await_pages.pop(task_id, None)
            if held is None:
                self._early_pages[task_id] = slot_mapping
                return
        for g in held:
            self._bind(g, slot_mapping)
        self.submit_batch(held)

    def wait(self, timeout: Optional[float] = None) -> List[CompletedOp]:
        if not self._ready.is_set():
            if timeout:
                self._ready.wait(timeout)
            if not self._ready.is_set():
                return []
        return self.engine.wait(timeout)

    def completion_fd(self) -> int:
        """-1 until the engine runs, or when its scheduler has no descriptor to poll."""
        if not self._ready.is_set() or not hasattr(self.engine, "completion_fd"):
            return -1
        return self.engine.completion_fd()

    def shutdown(self) -> None:
        self._stop = True
        with self._reg_cv:
            self._reg_cv.notify_all()
        if self._listener is not None:
            self._listener.stop()
            self._listener = None
        if self._init_thread is not None:
            self._init_thread.join(timeout=60)
        if self.engine is not None:
            self.engine.shutdown()
            self.engine = None
        if self.storage is not None:
            self.storage.shutdown()
            self.storage = None
        self._ready.clear()


# ------------------------------------------------------------------ other nodes / processes

def _remote_main(model_config, cache_config, cmd, res, qry, gpu_register_port, require_gpu) -> None:
    import signal
    from .common.debug import install_crash_diagnostics
    install_crash_diagnostics()
    signal.signal(signal.SIGINT, signal.SIG_IGN)
    node = TransferManagerOnRemote(model_config, cache_config, cmd, res, qry, require_gpu=require_gpu,
                                   gpu_register_port=gpu_register_port)
    signal.signal(signal.SIGTERM, lambda *_: node._stop.set())      # leave the serve loop, then unpin
    node.serve_forever()


class TransferManagerOnRemote:
    """Runs a TransferManager for this node's GPUs on behalf of a master node: graphs
    arrive on a ZeroMQ PULL socket, completions go back on a PUSH socket, readiness is
    answered on a REP socket (reference: flexkv/transfer_manager.py:529-908, ports
    5556-5558 at :1314-1343). The node keeps its own host pool; block ids in the graphs
    are the master's, applied to the same positions here."""

    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, command_endpoint: str,
                 result_endpoint: str, query_endpoint: str, require_gpu: bool = True,
                 gpu_register_port: Optional[str] = None) -> None:
        import zmq
        self.tm = TransferManager(model_config, cache_config, gpu_register_port, require_gpu=require_gpu)
        self._ctx = zmq.Context.instance()
        self._cmd = self._ctx.socket(zmq.PULL)
        self._cmd.setsockopt(zmq.LINGER, 0)
        self._cmd.bind(command_endpoint)
        self._res = self._ctx.socket(zmq.PUSH)
        self._res.setsockopt(zmq.LINGER, 0)
        self._res.connect(result_endpoint)
        self._qry = self._ctx.socket(zmq.REP)
        self._qry.setsockopt(zmq.LINGER, 0)
        self._qry.bind(query_endpoint)
        self._stop = threading.Event()

    def register_gpu(self, reg: GpuRegistration) -> None:
        self.tm.register_gpu(reg)

    @staticmethod
    def create_process(model_config: ModelConfig, cache_config: CacheConfig, command_endpoint: str,
                       result_endpoint: str, query_endpoint: str, gpu_register_port: Optional[str] = None,
                       require_gpu: bool = True):
        """Starts this node's transfer manager in a process of its own (spawn) and returns the process: local
        engine workers register their tensors at ``gpu_register_port``, the master drives it over the three
        endpoints (flexkv/transfer_manager.py:529-908 ``TransferManagerOnRemote.create_process``)."""
        import multiprocessing as mp
        p = mp.get_context("spawn").Process(target=_remote_main, name="flexkv-remote-transfer-manager", daemon=True,
                                            args=(model_config, cache_config, command_endpoint, result_endpoint,
                                                  query_endpoint, gpu_register_port, require_gpu))
        p.start()
        return p

    def serve_forever(self) -> None:
        import pickle
        import zmq
        self.tm.start()
        pump = threading.Thread(target=self._pump_results, name="flexkv-remote-results", daemon=True)
        pump.start()
        poller = zmq.Poller()
        poller.register(self._cmd, zmq.POLLIN)
        poller.register(self._qry, zmq.POLLIN)
        while not self._stop.is_set():
            for sock, _ in poller.poll(100):
                if sock is self._qry:
                    q = pickle.loads(self._qry.recv())
                    try:
                        ans = self.tm.is_ready() if q == "ready" else None
                    except RuntimeError as e:
                        ans = repr(e)
                    self._qry.send(pickle.dumps(ans))
                    continue
                kind, payload = pickle.loads(self._cmd.recv())
                if kind == "submit":
                    self.tm.submit_batch(payload)
                elif kind == "shutdown":
                    self._stop.set()
        pump.join(timeout=2)
        self.tm.shutdown()
        for s in (self._cmd, self._res, self._qry):
            s.close()

    def _pump_results(self) -> None:
        import pickle
        while not self._stop.is_set():
            done = self.tm.wait(timeout=0.05)
            if done:
                self._res.send(pickle.dumps(done))


class TransferManagerMultiNodeHandle:
    """Master-side handle of a TransferManagerOnRemote: same interface as an in-process
    TransferManager, so the task layer counts it as one more handle whose completions
    must arrive before a graph is finished (flexkv/transfer_manager.py:1279-1468)."""

    def __init__(self, command_endpoint: str, result_endpoint: str, query_endpoint: str,
                 rebind_gpu_blocks: bool = False) -> None:
        import zmq
        # rebind_gpu_blocks: the other node numbers its GPU pages itself; graphs go there with their GPU side
        # cleared and wait for that node's ranks to send the page list of the task (KVTPClient.set_slot_mapping)
        self.rebind_gpu_blocks = rebind_gpu_blocks
        self._ctx = zmq.Context.instance()
        self._cmd = self._ctx.socket(zmq.PUSH)
        self._cmd.setsockopt(zmq.LINGER, 0)
        self._cmd.connect(command_endpoint)
        self._res = self._ctx.socket(zmq.PULL)
        self._res.setsockopt(zmq.LINGER, 0)
        self._res.bind(result_endpoint)
        self._query_endpoint = query_endpoint
        self._lock = threading.Lock()

    def start(self) -> None:
        pass

    def is_ready(self) -> bool:
        import pickle
        import zmq
        q = self._ctx.socket(zmq.REQ)
        q.setsockopt(zmq.LINGER, 0)
        q.setsockopt(zmq.RCVTIMEO, 500)
        q.setsockopt(zmq.SNDTIMEO, 500)
        try:
            q.connect(self._query_endpoint)
            q.send(pickle.dumps("ready"))
            ans = pickle.loads(q.recv())
        except zmq.ZMQError:
            return False
        finally:
            q.close()
        if isinstance(ans, str):
            raise RuntimeError(f"remote transfer manager failed to start: {ans}")
        return bool(ans)

    def submit(self, graph: TransferOpGraph) -> None:
        self.submit_batch([graph])

    def submit_batch(self, graphs: List[TransferOpGraph]) -> None:
        import pickle
        if self.rebind_gpu_blocks:
            out = []
            for g in graphs:
                c = pickle.loads(pickle.dumps(g))          # this node's own graph keeps its binding
                if getattr(c, "task_id", None) is not None:
                    c.clear_gpu_blocks(force=True)
                    c.bind_task_id = c.task_id
                out.append(c)
            graphs = out
        with self._lock:
            self._cmd.send(pickle.dumps(("submit", graphs)))

    def wait(self, timeout: Optional[float] = None) -> List[CompletedOp]:
        import pickle
        if not self._res.poll(int((timeout or 0) * 1000)):
            return []
        out: List[CompletedOp] = []
        while self._res.poll(0):
            out.extend(pickle.loads(self._res.recv()))
        return out

    def set_metrics_collector(self, collector) -> None:
        pass

    def shutdown(self) -> None:
        import pickle
        try:
            with self._lock:
                self._cmd.send(pickle.dumps(("shutdown", None)))
        except Exception:  # noqa: BLE001
            pass
        self._cmd.close()
        self._res.close()
