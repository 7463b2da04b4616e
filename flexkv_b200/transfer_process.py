"""The data plane in a process of its own.

``TransferManagerProcessHandle`` has the interface of ``TransferManager`` and runs one in a child
process (spawn), for deployments that want the serving process shielded from the data plane: a
crash or a wedged GPU call in a worker cannot take the scheduler down, and pinned memory is
released by a process that can be killed. It follows the reference's discipline
(flexkv/transfer_manager.py:970-1272, flexkv/transfer/worker.py:189-239,342-383):

* commands and completions travel over one duplex pipe (pickled graphs down, completed ops up);
* the child notices the parent's death by EOF on the pipe and shuts down on its own;
* SIGINT is ignored in the child, SIGTERM raises ``SystemExit`` so that the ``finally`` block unpins;
  before unpinning, ``cuda.synchronize`` runs in a daemon thread with a time limit, so a wedged GPU
  cannot block the release of host memory;
* the parent notices the child's death the same way and reports every graph still in flight as
  FAILED (never a timeout), then removes the pool file the child may have left behind;
* ``faulthandler`` prints every thread's stack on a fatal signal (``common.debug.install_crash_diagnostics``).

GPU tensors reach the child as exported handles through the registration endpoint
(``gpu_register_port``), exactly as engine workers in other processes register.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import threading
import time
from typing import Dict, List, Optional

from .common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from .common.debug import flexkv_logger
from .common.transfer import CompletedOp, TransferOpGraph


def _bounded_cuda_synchronize(limit_s: float) -> bool:
    """``torch.cuda.synchronize`` on every device in a daemon thread; False when it did not return in time."""
    done = threading.Event()

    def run() -> None:
        try:
            import torch
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                for d in range(torch.cuda.device_count()):
                    torch.cuda.synchronize(d)
        except Exception:  # noqa: BLE001
            pass
        done.set()
    threading.Thread(target=run, name="flexkv-sync-before-unpin", daemon=True).start()
    return done.wait(limit_s)


def _child_main(conn, model_config: ModelConfig, cache_config: CacheConfig, gpu_register_port: Optional[str],
                require_gpu: bool, sync_limit_s: float) -> None:
    from .common.debug import install_crash_diagnostics
    from .transfer_manager import TransferManager
    install_crash_diagnostics()
    signal.signal(signal.SIGINT, signal.SIG_IGN)

    def on_term(signum, frame):     # noqa: ARG001
        raise SystemExit(0)
    signal.signal(signal.SIGTERM, on_term)
    tm = TransferManager(model_config, cache_config, gpu_register_port, require_gpu=require_gpu)
    stop = threading.Event()
    send_lock = threading.Lock()

    def send(msg) -> None:
        with send_lock:
            conn.send(msg)

    def pump() -> None:
        announced = False
        while not stop.is_set():
            try:
                if not announced:
                    if tm.is_ready():
                        st = tm.storage
                        send(("ready", dict(pool_file=getattr(st, "host_backing_file", "") or "", pid=os.getpid())))
                        announced = True
                    else:
                        time.sleep(0.01)
                        continue
                done = tm.wait(timeout=0.05)
                if done:
                    send(("done", done))
            except RuntimeError as e:          # initialisation failed
                send(("error", repr(e)))
                return
            except (OSError, EOFError, BrokenPipeError):
                return
    try:
        tm.start()
        th = threading.Thread(target=pump, name="flexkv-tm-results", daemon=True)
        th.start()
        while True:
            if not conn.poll(0.2):
                continue
            try:
                msg = conn.recv()
            except (EOFError, OSError):
                flexkv_logger.warning("transfer manager process: the parent is gone, shutting down")
                break
            kind = msg[0]
            if kind == "submit":
                tm.submit_batch(msg[1])
            elif kind == "suspend":
                send(("suspended", msg[1], tm.suspend_gpu_mappings(msg[2], msg[3])))
            elif kind == "resume":
                tm.resume_gpu_mappings(msg[1], None)
            elif kind == "shutdown":
                break
    finally:
        stop.set()
        if not _bounded_cuda_synchronize(sync_limit_s):
            flexkv_logger.error("GPU did not quiesce in %.0f s; unpinning host memory anyway", sync_limit_s)
        try:
            tm.shutdown()
        except Exception:  # noqa: BLE001
            flexkv_logger.exception("transfer manager process: shutdown failed")
        try:
            send(("bye",))
            conn.close()
        except Exception:  # noqa: BLE001
            pass


class TransferManagerProcessHandle:
    """Drop-in for ``TransferManager`` whose work happens in a child process."""

    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, gpu_register_port: Optional[str] = None,
                 require_gpu: bool = True, sync_limit_s: float = 30.0) -> None:
        self.model_config, self.cache_config = model_config, cache_config
        self.gpu_register_port = gpu_register_port or f"ipc:///tmp/flexkv_gpu_register_{os.getpid()}_{id(self) & 0xffff}"
        self.require_gpu = require_gpu
        self.sync_limit_s = sync_limit_s
        self.engine = None          # lives in the child
        self.storage = None
        self._proc: Optional[mp.Process] = None
        self._conn = None
        self._reader: Optional[threading.Thread] = None
        self._ready = threading.Event()
        self._error: Optional[str] = None
        self._dead = threading.Event()
        self._cv = threading.Condition()
        self._done: List[CompletedOp] = []
        self._inflight: Dict[int, bool] = {}       # graph ids submitted and not reported finished
        self._suspend_waiters: Dict[int, list] = {}
        self._pool_file = ""
        self._tp_clients = []
        self._seq = 0

    # ---- registration: tensors are exported and sent to the child's registration endpoint ------------
    def register_gpu_tensors(self, tensors, gpu_layout, tp_rank=0, pp_rank=0, dp_client_id=0, group_id=-1) -> None:
        from .server.client import KVTPClient
        dev = (tensors[0].device.index or 0) if tensors[0].is_cuda else -1
        c = KVTPClient(self.gpu_register_port, dp_client_id, dev, pp_rank=pp_rank, tp_rank=tp_rank)
        c.register_to_server(tensors, gpu_layout, group_id=group_id)
        self._tp_clients.append(c)

    def register_gpu(self, reg) -> None:
        raise RuntimeError("the data plane runs in another process: register tensors, not addresses "
                           "(register_gpu_tensors, or KVTPClient.register_to_server from the engine worker)")

    register_swa = register_gpu

    # ---- lifecycle ----------------------------------------------------------------------------------
    def start(self) -> None:
        if self._proc is not None:
            return
        ctx = mp.get_context("spawn")
        parent, child = ctx.Pipe(duplex=True)
        self._conn = parent
        self._proc = ctx.Process(target=_child_main, name="flexkv-transfer-manager",
                                 args=(child, self.model_config, self.cache_config, self.gpu_register_port,
                                       self.require_gpu, self.sync_limit_s), daemon=True)
        self._proc.start()
        child.close()                       # EOF reaches each side when the other one dies
        self._reader = threading.Thread(target=self._read_loop, name="flexkv-tm-reader", daemon=True)
        self._reader.start()

    def _read_loop(self) -> None:
        try:
            while True:
                msg = self._conn.recv()
                kind = msg[0]
                if kind == "ready":
                    self._pool_file = msg[1].get("pool_file", "")
                    self._ready.set()
                elif kind == "done":
                    with self._cv:
                        for c in msg[1]:
                            if c.is_graph_completed():
                                self._inflight.pop(c.graph_id, None)
                        self._done.extend(msg[1])
                        self._cv.notify_all()
                elif kind == "suspended":
                    w = self._suspend_waiters.pop(msg[1], None)
                    if w is not None:
                        w[1] = bool(msg[2])
                        w[0].set()
                elif kind == "error":
                    self._error = msg[1]
                elif kind == "bye":
                    break
        except (EOFError, OSError):
            pass
        self._on_child_gone()

    def _on_child_gone(self) -> None:
        """The child ended (asked to, or killed): whatever it still owed is reported as failed."""
        self._dead.set()
        if self._pool_file:
            try:
                os.unlink(self._pool_file)     # a killed child cannot remove its pool file itself
            except OSError:
                pass
        with self._cv:
            lost = list(self._inflight)
            self._inflight.clear()
            for gid in lost:
                self._done.append(CompletedOp.graph_done(gid, success=False))
            self._cv.notify_all()
        if lost:
            flexkv_logger.error("transfer manager process ended with %d graph(s) in flight: reported as failed",
                                len(lost))
        for w in list(self._suspend_waiters.values()):
            w[0].set()

    def is_ready(self) -> bool:
        if self._error is not None:
            raise RuntimeError(f"transfer manager failed to start: {self._error}")
        if self._dead.is_set() and not self._ready.is_set():
            raise RuntimeError("transfer manager process ended before it became ready")
        return self._ready.is_set() and not self._dead.is_set()

    def alive(self) -> bool:
        return self._proc is not None and self._proc.is_alive() and not self._dead.is_set()

    @property
    def pid(self) -> Optional[int]:
        return self._proc.pid if self._proc is not None else None

    def set_metrics_collector(self, collector) -> None:
        pass        # the child exports its own counters

    # ---- work ---------------------------------------------------------------------------------------
    def submit(self, graph: TransferOpGraph) -> None:
        self.submit_batch([graph])

    def submit_batch(self, graphs: List[TransferOpGraph]) -> None:
        with self._cv:
            if self._dead.is_set():
                for g in graphs:
                    self._done.append(CompletedOp.graph_done(g.graph_id, success=False))
                self._cv.notify_all()
                return
            for g in graphs:
                self._inflight[g.graph_id] = True
        try:
            self._conn.send(("submit", graphs))
        except (OSError, BrokenPipeError, ValueError):
            self._on_child_gone()

    def wait(self, timeout: Optional[float] = None) -> List[CompletedOp]:
        with self._cv:
            if not self._done and (timeout is None or timeout > 0):
                self._cv.wait(timeout)
            out, self._done = self._done, []
        return out

    def suspend_gpu_mappings(self, dp_client_id: Optional[int] = None, timeout: float = 60.0) -> bool:
        self._seq += 1
        w = [threading.Event(), False]
        self._suspend_waiters[self._seq] = w
        self._conn.send(("suspend", self._seq, dp_client_id, timeout))
        w[0].wait(timeout + 5)
        return bool(w[1])

    def resume_gpu_mappings(self, dp_client_id: Optional[int] = None, new_registrations=None) -> None:
        if new_registrations:
            raise RuntimeError("re-created tensors are re-registered through KVTPClient in process mode")
        self._conn.send(("resume", dp_client_id))

    def shutdown(self) -> None:
        if self._proc is None:
            return
        try:
            self._conn.send(("shutdown",))
        except (OSError, BrokenPipeError, ValueError):
            pass
        self._proc.join(timeout=GLOBAL_CONFIG_FROM_ENV.transfer_manager_shutdown_timeout_s)
        if self._proc.is_alive():
            flexkv_logger.error("transfer manager process did not exit in time: SIGTERM")
            self._proc.terminate()
            self._proc.join(timeout=self.sync_limit_s + 10)
            if self._proc.is_alive():
                self._proc.kill()
                self._proc.join(timeout=5)
        self._proc = None
        for c in self._tp_clients:
            try:
                c.shutdown()
            except Exception:  # noqa: BLE001
                pass
        self._tp_clients = []
