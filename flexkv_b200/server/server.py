"""KV server: one process (or thread) that owns the shared index and the data
plane for several data-parallel ranks / engine instances; clients talk to it
over ZeroMQ (flexkv/server/server.py:147-510). Requests arrive on one PULL
socket and are dispatched through a handler table; every client gets its
responses on its own PUSH socket."""
from __future__ import annotations

import multiprocessing as mp
import pickle
import threading
import time
from typing import Any, Callable, Dict, Optional

import zmq

from ..common.config import CacheConfig, ModelConfig
from ..common.debug import flexkv_logger
from . import request as R
from .utils import get_zmq_socket


PARKED_PUMP_S = 0.0002     # longest a new request waits behind the completion queue while waits are parked


class KVServer:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, recv_endpoint: str,
                 gpu_register_port: Optional[str] = None, require_gpu: Optional[bool] = None) -> None:
        from ..kvtask import KVTaskEngine
        from ..transfer_manager import TransferManager
        import torch
        self.model_config, self.cache_config = model_config, cache_config
        self.recv_endpoint = recv_endpoint
        self._ctx = zmq.Context.instance()
        self._recv = get_zmq_socket(self._ctx, zmq.PULL, recv_endpoint, bind=True)
        self._clients: Dict[int, zmq.Socket] = {}
        if require_gpu is None:
            require_gpu = torch.cuda.is_available()
        self.transfer_manager = TransferManager(model_config, cache_config, gpu_register_port, require_gpu=require_gpu)
        self.engine = KVTaskEngine(model_config, cache_config, transfer_handles=[self.transfer_manager])
        self._running = False
        self._handlers: Dict[type, Callable[[Any], Optional[R.Response]]] = {
            R.RegisterDPClientRequest: self._on_register_dp,
            R.IsReadyRequest: self._on_is_ready,
            R.PutRequest: self._on_put,
            R.GetRequest: self._on_get,
            R.PrefetchRequest: self._on_prefetch,
            R.LaunchRequest: self._on_launch,
            R.CancelRequest: self._on_cancel,
            R.WaitRequest: self._on_wait,
            R.ResetRequest: self._on_reset,
            R.PublishGpuBlocksRequest: self._on_publish,
            R.WithdrawGpuBlocksRequest: self._on_withdraw,
            R.ShutdownRequest: self._on_shutdown,
            R.UnregisterDPClientRequest: self._on_unregister_dp,
        }

    # ---- process / thread front ends ---------------------------------------------------
    @classmethod
    def create_server(cls, model_config, cache_config, recv_endpoint, gpu_register_port=None, mode: str = "thread",
                      require_gpu: Optional[bool] = None) -> "ServerHandle":
        """`thread` runs the server inside this process (it shares the caller's CUDA
        context, which is what single-node deployments want); `process` spawns it."""
        if mode == "process":
            ctx = mp.get_context("spawn")
            ready = ctx.Event()
            p = ctx.Process(target=_server_main, args=(model_config, cache_config, recv_endpoint, gpu_register_port,
                                                       ready, require_gpu), daemon=True)
            p.start()
            if not ready.wait(120):
                raise RuntimeError("KV server did not come up")
            return ServerHandle(process=p, endpoint=recv_endpoint)
        srv = cls(model_config, cache_config, recv_endpoint, gpu_register_port, require_gpu)
        t = threading.Thread(target=srv.run, name="flexkv-server", daemon=True)
        t.start()
        return ServerHandle(thread=t, server=srv, endpoint=recv_endpoint)

    _leaving: list = []

    def run(self) -> None:
        self._leaving = []
        self.engine.start()
        self._running = True
        poller = zmq.Poller()
        poller.register(self._recv, zmq.POLLIN)
        self._parked = []
        self._completion_fds: list = []
        self._probe_fds = 50
        while self._running:
            # a blocking wait of one client must not hold up the others: it is parked and answered from here
            # once its tasks are done (or its time is up); requests keep being served meanwhile
            # The loop sleeps until a request OR a completion arrives: the data plane's completion queue has a
            # descriptor the poller can watch. Where it has none (data plane in another process, Python
            # scheduler) and somebody waits for tasks, look for a request without blocking and else block on the
            # completion queue for PARKED_PUMP_S at a time.
            if not self._completion_fds and self._probe_fds > 0:
                fds = self.engine.completion_fds()
                if fds:
                    for fd in fds:
                        poller.register(fd, zmq.POLLIN)
                    self._completion_fds = fds
                elif fds is None or self.engine.is_ready():
                    self._probe_fds -= 1               # handles without a descriptor: stop asking after a while
            if self._parked:
                if self._completion_fds:
                    next_deadline = min(d for _, d in self._parked)
                    ms = max(0, min(100, int((next_deadline - time.monotonic()) * 1000) + 1))
                    ready = dict(poller.poll(ms))
                    if self._recv not in ready:
                        self._answer_parked_waits()      # applies the completions, which also empties the descriptor
                        continue
                elif not dict(poller.poll(0)):
                    self.engine.pump(PARKED_PUMP_S)
                    self._answer_parked_waits()
                    continue
            else:
                ready = dict(poller.poll(100))
                if self._recv not in ready:
                    if ready:
                        self.engine.pump(0.0)    # completions nobody waits for yet: apply them, which empties the descriptor
                    continue
            try:
                req = pickle.loads(self._recv.recv())
            except Exception:  # noqa: BLE001
                flexkv_logger.exception("undecodable request")
                continue
            handler = self._handlers.get(type(req))
            if handler is None:
                flexkv_logger.error("no handler for %s", type(req).__name__)
                continue
            try:
                rsp = handler(req)
            except Exception as e:  # noqa: BLE001
                flexkv_logger.exception("request %s failed", type(req).__name__)
                rsp = R.Response(req.dp_client_id, req.seq, error=repr(e))
            if rsp is not None:
                self._reply(rsp)
            self._answer_parked_waits()
            while self._leaving:                       # after the answer went out
                gone = self._clients.pop(self._leaving.pop(), None)
                if gone is not None:
                    gone.close(linger=1000)
        # waits still parked get their answer (what has finished, TIMEOUT for the rest) before the sockets close
        for q, _ in self._parked:
            try:
                self._reply(R.Response(q.dp_client_id, q.seq, status=self.engine.wait(q.task_ids, 0.0, q.completely)))
            except Exception:  # noqa: BLE001
                pass
        self._parked = []
        self.engine.shutdown()
        for s in self._clients.values():
            s.close(linger=1000)
        self._recv.close()

    def _reply(self, rsp: R.Response) -> None:
        sock = self._clients.get(rsp.dp_client_id)
        if sock is not None:
            sock.send(pickle.dumps(rsp, protocol=pickle.HIGHEST_PROTOCOL))

    # ---- handlers -------------------------------------------------------------------------
    def _on_register_dp(self, q: R.RegisterDPClientRequest):
        old = self._clients.pop(q.dp_client_id, None)
        if old is not None:
            old.close()
        self._clients[q.dp_client_id] = get_zmq_socket(self._ctx, zmq.PUSH, q.client_recv_port, bind=False)
        return R.Response(q.dp_client_id, q.seq, ready=True)

    def _on_is_ready(self, q):
        return R.Response(q.dp_client_id, q.seq, ready=self.engine.is_ready())

    def _on_put(self, q: R.PutRequest):
        if q.match_only:
            tid, mask = self.engine.put_match(q.token_ids, q.token_mask, q.dp_client_id, q.namespace)
        else:
            tid, mask = self.engine.put_async(q.token_ids, q.slot_mapping, q.token_mask, q.dp_client_id, q.namespace)
        return R.Response(q.dp_client_id, q.seq, task_id=tid, mask=mask)

    def _on_get(self, q: R.GetRequest):
        if q.match_only:
            tid, mask = self.engine.get_match(q.token_ids, q.token_mask, q.dp_client_id, q.cpu_only, q.namespace,
                                              q.swa_aware)
        else:
            tid, mask = self.engine.get_async(q.token_ids, q.slot_mapping, q.token_mask, q.dp_client_id, q.namespace)
        return R.Response(q.dp_client_id, q.seq, task_id=tid, mask=mask)

    def _on_prefetch(self, q: R.PrefetchRequest):
        return R.Response(q.dp_client_id, q.seq, task_id=self.engine.prefetch_async(q.token_ids, q.dp_client_id,
                                                                                    q.namespace, q.swa_aware))

    def _on_launch(self, q: R.LaunchRequest):
        ids = self.engine.launch_tasks(q.task_ids, q.slot_mappings, as_batch=q.as_batch,
                                       layerwise_transfer=q.layerwise_transfer, counter_id=q.counter_id)
        return R.Response(q.dp_client_id, q.seq, task_ids=ids)

    def _on_cancel(self, q: R.CancelRequest):
        self.engine.cancel_tasks(q.task_ids)
        return R.Response(q.dp_client_id, q.seq, value=True)

    def _on_wait(self, q: R.WaitRequest):
        if q.try_wait:
            return R.Response(q.dp_client_id, q.seq, status=self.engine.try_wait(q.task_ids))
        if not self.engine.wait_would_return_now(q.task_ids, q.completely):
            self._parked.append((q, time.monotonic() + float(q.timeout)))
            return None
        return R.Response(q.dp_client_id, q.seq, status=self.engine.wait(q.task_ids, 0.0, q.completely))

    def _answer_parked_waits(self) -> None:
        if not self._parked:
            return
        still, now = [], time.monotonic()
        for q, deadline in self._parked:
            try:
                if now >= deadline or self.engine.wait_would_return_now(q.task_ids, q.completely):
                    # unfinished tasks of a wait whose time is up come back as TIMEOUT, as from a blocking wait
                    self._reply(R.Response(q.dp_client_id, q.seq, status=self.engine.wait(q.task_ids, 0.0, q.completely)))
                else:
                    still.append((q, deadline))
            except Exception as e:  # noqa: BLE001
                flexkv_logger.exception("parked wait failed")
                self._reply(R.Response(q.dp_client_id, q.seq, error=repr(e)))
        self._parked = still

    def _on_reset(self, q):
        self.engine.reset_cache()
        return R.Response(q.dp_client_id, q.seq, value=True)

    def _on_publish(self, q: R.PublishGpuBlocksRequest):
        n = self.engine.publish_gpu_blocks(q.token_ids, q.slot_mapping, q.dp_client_id, q.namespace)
        return R.Response(q.dp_client_id, q.seq, value=n)

    def _on_withdraw(self, q: R.WithdrawGpuBlocksRequest):
        return R.Response(q.dp_client_id, q.seq, value=self.engine.withdraw_gpu_blocks(q.gpu_block_ids, q.dp_client_id))

    def _on_unregister_dp(self, q: R.UnregisterDPClientRequest):
        """Detaches one client: its tasks that were matched but never launched give their reservations back, its
        published GPU blocks leave the peer directory, and its reply socket is closed after this answer."""
        stale = [tid for tid, t in list(self.engine.tasks.items())
                 if getattr(t, "dp_id", None) == q.dp_client_id and t.status.name == "UNREADY"]
        if stale:
            self.engine.cancel_tasks(stale)
        pd = self.engine.cache_engine.peer_directory
        if pd is not None:
            pd.clear_rank(q.dp_client_id)
        self._leaving.append(q.dp_client_id)
        return R.Response(q.dp_client_id, q.seq, value=len(stale))

    def _on_shutdown(self, q):
        self._running = False
        return R.Response(q.dp_client_id, q.seq, value=True)


def _server_main(model_config, cache_config, endpoint, gpu_register_port, ready, require_gpu) -> None:
    import signal
    signal.signal(signal.SIGINT, signal.SIG_IGN)            # the parent decides when to stop
    signal.signal(signal.SIGTERM, lambda *_: (_ for _ in ()).throw(SystemExit(0)))
    srv = KVServer(model_config, cache_config, endpoint, gpu_register_port, require_gpu)
    ready.set()
    try:
        srv.run()
    finally:
        try:
            srv.engine.shutdown()
        except Exception:  # noqa: BLE001
            pass


class ServerHandle:
    def __init__(self, endpoint: str, process=None, thread=None, server: Optional[KVServer] = None) -> None:
        self.endpoint, self.process, self.thread, self.server = endpoint, process, thread, server

    def shutdown(self, timeout: float = 30.0) -> None:
        ctx = zmq.Context.instance()
        s = get_zmq_socket(ctx, zmq.PUSH, self.endpoint, bind=False)
        s.send(pickle.dumps(R.ShutdownRequest(dp_client_id=-1)))
        time.sleep(0.05)
        s.close()
        if self.thread is not None:
            self.thread.join(timeout)
        if self.process is not None:
            self.process.join(timeout)
            if self.process.is_alive():
                self.process.terminate()
