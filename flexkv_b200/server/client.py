"""Clients of the KV server: ``KVDPClient`` (one per data-parallel rank, mirrors
the KVManager API) and ``KVTPClient`` (one per engine worker, registers that
worker's GPU KV tensors) — flexkv/server/client.py:39-288,290-517."""
from __future__ import annotations

import pickle
import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import zmq

from ..common.config import ModelConfig
from ..common.debug import flexkv_logger
from ..common.memory_handle import TensorSharedHandle
from ..common.request import KVResponse
from ..common.storage import KVCacheLayout
from . import request as R
from .utils import get_zmq_socket, unique_ipc_endpoint


class KVDPClient:
    def __init__(self, server_recv_port: str, model_config: ModelConfig, dp_client_id: int = 0,
                 request_timeout: float = 120.0) -> None:
        self.dp_client_id = dp_client_id
        self.model_config = model_config
        self.request_timeout = request_timeout
        self._ctx = zmq.Context.instance()
        self._send = get_zmq_socket(self._ctx, zmq.PUSH, server_recv_port, bind=False)
        self._recv_endpoint = unique_ipc_endpoint(f"flexkv_dp{dp_client_id}")
        self._recv = get_zmq_socket(self._ctx, zmq.PULL, self._recv_endpoint, bind=True)
        self._seq = 0
        self._lock = threading.Lock()
        self._registered = False

    def _call(self, req: R.Request, timeout: Optional[float] = None) -> R.Response:
        with self._lock:
            self._seq += 1
            req.dp_client_id, req.seq = self.dp_client_id, self._seq
            self._send.send(pickle.dumps(req, protocol=pickle.HIGHEST_PROTOCOL))
            deadline = time.monotonic() + (timeout if timeout is not None else self.request_timeout)
            while True:
                left = deadline - time.monotonic()
                if left <= 0 or not self._recv.poll(int(left * 1000)):
                    raise TimeoutError(f"KV server did not answer {type(req).__name__}")
                rsp: R.Response = pickle.loads(self._recv.recv())
                if rsp.seq != self._seq:
                    continue                      # a stale answer to a request that timed out earlier
                if rsp.error:
                    raise RuntimeError(f"KV server: {rsp.error}")
                return rsp

    def start_server_and_register(self) -> None:
        if not self._registered:
            self._call(R.RegisterDPClientRequest(client_recv_port=self._recv_endpoint))
            self._registered = True

    def is_ready(self) -> bool:
        self.start_server_and_register()
        return bool(self._call(R.IsReadyRequest()).ready)

    def put_async(self, token_ids, slot_mapping, token_mask=None, namespace=None) -> int:
        return self._call(R.PutRequest(token_ids=token_ids, slot_mapping=slot_mapping, token_mask=token_mask,
                                       namespace=namespace)).task_id

    def put_match(self, token_ids, token_mask=None, namespace=None) -> Tuple[int, np.ndarray]:
        r = self._call(R.PutRequest(token_ids=token_ids, token_mask=token_mask, namespace=namespace, match_only=True))
        return r.task_id, r.mask

    def get_async(self, token_ids, slot_mapping, token_mask=None, namespace=None) -> int:
        return self._call(R.GetRequest(token_ids=token_ids, slot_mapping=slot_mapping, token_mask=token_mask,
                                       namespace=namespace)).task_id

    def get_match(self, token_ids, token_mask=None, cpu_only=False, namespace=None, swa_aware=False):
        r = self._call(R.GetRequest(token_ids=token_ids, token_mask=token_mask, namespace=namespace, match_only=True,
                                    cpu_only=cpu_only, swa_aware=swa_aware))
        return r.task_id, r.mask

    def prefetch_async(self, token_ids, namespace=None, swa_aware=False) -> int:
        return self._call(R.PrefetchRequest(token_ids=token_ids, namespace=namespace, swa_aware=swa_aware)).task_id

    def launch_tasks(self, task_ids, slot_mappings, swa_slot_mappings=None, as_batch=False, layerwise_transfer=False,
                     counter_id=0) -> List[int]:
        return self._call(R.LaunchRequest(task_ids=list(task_ids), slot_mappings=list(slot_mappings),
                                          as_batch=as_batch, layerwise_transfer=layerwise_transfer,
                                          counter_id=counter_id)).task_ids

    def cancel_tasks(self, task_ids) -> None:
        self._call(R.CancelRequest(task_ids=list(task_ids)))

    def wait(self, task_ids=None, timeout: float = 20.0, completely: bool = False, *, wait_task_ids=None,
             wait_timeout: Optional[float] = None) -> Dict[int, KVResponse]:
        """``wait_task_ids`` / ``wait_timeout`` are the reference's names for the first two arguments."""
        task_ids = wait_task_ids if task_ids is None else task_ids
        timeout = timeout if wait_timeout is None else float(wait_timeout)
        return self._call(R.WaitRequest(task_ids=list(task_ids), timeout=timeout, completely=completely),
                          timeout=timeout + self.request_timeout).status

    def try_wait(self, task_ids=None, *, try_wait_task_ids=None) -> Dict[int, KVResponse]:
        task_ids = try_wait_task_ids if task_ids is None else task_ids
        return self._call(R.WaitRequest(task_ids=list(task_ids), try_wait=True)).status

    def register_to_server(self, model_config=None, client_recv_port: Optional[str] = None) -> None:
        """The reference's name for joining the server; the reply endpoint is this client's own."""
        self.start_server_and_register()

    def reset(self) -> None:
        self._call(R.ResetRequest())

    def publish_gpu_blocks(self, token_ids, slot_mapping, namespace=None) -> int:
        return self._call(R.PublishGpuBlocksRequest(token_ids=token_ids, slot_mapping=slot_mapping,
                                                    namespace=namespace)).value

    def withdraw_gpu_blocks(self, gpu_block_ids) -> List[int]:
        return self._call(R.WithdrawGpuBlocksRequest(gpu_block_ids=gpu_block_ids)).value

    def unregister(self) -> int:
        """Leaves the shared server (which keeps running for the other clients): tasks of this client that were
        matched but never launched are cancelled there. Returns how many."""
        if not self._registered:
            return 0
        n = int(self._call(R.UnregisterDPClientRequest(), timeout=10.0).value or 0)
        self._registered = False
        return n

    def shutdown(self) -> None:
        try:
            self.unregister()
        except Exception:  # noqa: BLE001 - the server may already be gone
            pass
        self._send.close()
        self._recv.close()


class KVTPClient:
    """Registers one engine worker's GPU KV tensors with the process that runs the
    data plane (address handles in the same process, CUDA IPC across processes)."""

    def __init__(self, gpu_register_port: str, dp_client_id: int = 0, device_id: int = 0,
                 intra_client_id: Optional[int] = None, tp_rank: int = 0, pp_rank: int = 0) -> None:
        self.dp_client_id, self.device_id = dp_client_id, device_id
        self.tp_rank, self.pp_rank = tp_rank, pp_rank
        self.intra_client_id = tp_rank if intra_client_id is None else intra_client_id
        if intra_client_id is not None and tp_rank == 0:
            self.tp_rank = intra_client_id
        self._ctx = zmq.Context.instance()
        self._sock = get_zmq_socket(self._ctx, zmq.PUSH, gpu_register_port, bind=False)
        # a registration must survive a client that is dropped right after sending it (the connection to the
        # data plane is made asynchronously): queued messages are flushed for up to 10 s after close
        self._sock.setsockopt(zmq.LINGER, 10000)
        self._handles: List[TensorSharedHandle] = []

    def register_to_server(self, kv_caches: Sequence[torch.Tensor], kv_layout: KVCacheLayout,
                           mode: Optional[str] = None, group_id: int = -1, layer_groups=None, *,
                           override_device_id: Optional[int] = None, gpu_layouts=None, handles_per_group=None,
                           swa_caches=None, swa_layout=None, swa_layer_groups=None, swa_gpu_layouts=None,
                           swa_handles_per_group=None, resume: bool = False) -> None:
        """``group_id``: layer group of a multi-group cache; call once per group. ``layer_groups``: the
        ``LayerGroupSpec`` list, for engines whose worker only learns the groups from its tensors (the data
        plane adopts the first list it receives when its own configuration names none;
        flexkv/transfer_manager.py:154-161).

        The keyword-only arguments are the one-call form engine integrations written for the reference use
        (flexkv/server/client.py:366-470): ``handles_per_group[g]`` / ``gpu_layouts[g]`` register every layer
        group at once, ``swa_caches`` (or ``swa_handles_per_group``: window pages first, then the state
        sidecars) the sliding-window pool, ``override_device_id`` replaces this client's device id, and
        ``resume`` re-registers after the engine re-created its tensors (sleep / wake)."""
        if override_device_id is not None:
            self.device_id = int(override_device_id)
        if swa_handles_per_group is not None or swa_gpu_layouts is not None or swa_layer_groups is not None:
            if swa_handles_per_group is None or swa_gpu_layouts is None or swa_layer_groups is None or not \
                    (len(swa_handles_per_group) == len(swa_gpu_layouts) == len(swa_layer_groups)):
                raise ValueError("swa_layer_groups, swa_gpu_layouts and swa_handles_per_group go together, "
                                 "one entry per group")
        if handles_per_group is not None:
            if gpu_layouts is None or len(gpu_layouts) != len(handles_per_group):
                raise ValueError("handles_per_group needs one gpu layout per group")
            if resume:
                first, rest = handles_per_group[0], list(zip(handles_per_group[1:], gpu_layouts[1:],
                                                            range(1, len(handles_per_group))))
                if not self.resume_gpu_mappings(first, gpu_layouts[0], mode, 0, rest):
                    raise RuntimeError("the data plane did not take the re-created tensors")
            else:
                for g, (tensors, layout) in enumerate(zip(handles_per_group, gpu_layouts)):
                    self.register_to_server(tensors, layout, mode, g, layer_groups if g == 0 else None)
        elif resume:
            if not self.resume_gpu_mappings(kv_caches, kv_layout, mode, group_id):
                raise RuntimeError("the data plane did not take the re-created tensors")
        if swa_handles_per_group is not None:
            for g, tensors in enumerate(swa_handles_per_group):
                self.register_swa_to_server(tensors, g, mode)
        elif swa_caches is not None:
            self.register_swa_to_server(swa_caches, 0, mode)
        if handles_per_group is not None or resume:
            return
        handles = [TensorSharedHandle.export(t, mode) for t in kv_caches]
        self._handles = self._handles + handles if group_id > 0 else handles
        req = R.RegisterTPClientRequest(self.dp_client_id, self.intra_client_id, self.device_id, handles,
                                        kv_layout, pp_rank=self.pp_rank, tp_rank=self.tp_rank, group_id=group_id,
                                        layer_groups=layer_groups)
        self._sock.send(pickle.dumps(req, protocol=pickle.HIGHEST_PROTOCOL))
        flexkv_logger.info("sent GPU registration: dp %d rank %d, %d tensors", self.dp_client_id,
                           self.intra_client_id, len(kv_caches))

    def set_slot_mapping(self, task_id: int, slot_mapping) -> None:
        """Tells the data plane of THIS node which GPU pages this node's ranks use for ``task_id`` (a task
        planned on the master node of a group that spans nodes; the graph waits there for this message)."""
        import numpy as np
        req = R.SlotMappingRequest(int(task_id), np.ascontiguousarray(np.asarray(slot_mapping), dtype=np.int64),
                                   self.dp_client_id)
        self._sock.send(pickle.dumps(req, protocol=pickle.HIGHEST_PROTOCOL))

    def register_swa_to_server(self, page_tensors: Sequence[torch.Tensor], group_id: int = 0,
                               mode: Optional[str] = None) -> None:
        """Sliding-window pages of this rank (one ``[num_pages, ...]`` tensor per window layer); ``group_id``
        g >= 1 names the g-th sidecar group of ``SWAPoolConfig.sidecar_groups``. The data plane waits for
        these when ``SWAPoolConfig.wait_for_registration`` is set."""
        handles = [TensorSharedHandle.export(t, mode) for t in page_tensors]
        self._swa_handles = getattr(self, "_swa_handles", []) + handles
        req = R.RegisterTPClientRequest(self.dp_client_id, self.intra_client_id, self.device_id, handles, None,
                                        pp_rank=self.pp_rank, tp_rank=self.tp_rank, group_id=int(group_id),
                                        is_swa=True)
        self._sock.send(pickle.dumps(req, protocol=pickle.HIGHEST_PROTOCOL))

    # ---- sleep / wake (vLLM sleep mode) ----------------------------------------------------
    def _control(self, action: str, registration=None, timeout: float = 60.0, more=None) -> bool:
        import os
        import uuid
        ep = f"ipc:///tmp/flexkv_ctl_{os.getpid()}_{uuid.uuid4().hex[:8]}"
        reply = get_zmq_socket(self._ctx, zmq.PULL, ep, bind=True)
        try:
            req = R.GpuControlRequest(self.dp_client_id, action, ep, registration, timeout, more or None)
            self._sock.send(pickle.dumps(req, protocol=pickle.HIGHEST_PROTOCOL))
            if not reply.poll(int((timeout + 5) * 1000)):
                return False
            return bool(pickle.loads(reply.recv()))
        finally:
            reply.close()
            try:
                os.unlink(ep[len("ipc://"):])
            except OSError:
                pass

    def suspend_gpu_mappings(self, timeout: float = 60.0) -> bool:
        """Blocks until the data plane no longer touches (or maps) this client's KV tensors."""
        return self._control("suspend", None, timeout)

    def resume_gpu_mappings(self, kv_caches: Optional[Sequence[torch.Tensor]] = None,
                            kv_layout: Optional[KVCacheLayout] = None, mode: Optional[str] = None,
                            group_id: int = -1, more_groups: Optional[Sequence[tuple]] = None) -> bool:
        """Hands over the re-created tensors (omit them when the memory came back at the old addresses). A
        multi-group cache passes its first group here with its ``group_id`` and the others as
        ``more_groups = [(tensors, layout, group_id), ...]``."""
        reg, more = None, []
        if kv_caches is not None:
            self._handles = [TensorSharedHandle.export(t, mode) for t in kv_caches]
            reg = R.RegisterTPClientRequest(self.dp_client_id, self.intra_client_id, self.device_id, self._handles,
                                            kv_layout, pp_rank=self.pp_rank, tp_rank=self.tp_rank, group_id=group_id)
            for tensors, layout, gid in (more_groups or []):
                handles = [TensorSharedHandle.export(t, mode) for t in tensors]
                self._handles = self._handles + handles
                more.append(R.RegisterTPClientRequest(self.dp_client_id, self.intra_client_id, self.device_id, handles,
                                                      layout, pp_rank=self.pp_rank, tp_rank=self.tp_rank,
                                                      group_id=int(gid)))
        return self._control("resume", reg, more=more)

    def shutdown(self) -> None:
        self._sock.close()
