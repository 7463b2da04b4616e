"""GPU registration over ZeroMQ: engine workers PUSH their tensor handles, the
data plane's owner PULLs them and opens the memory
(flexkv/transfer_manager.py:77-83,317-357; flexkv/server/client.py:366-496)."""
from __future__ import annotations

import pickle
import threading
from typing import Callable, Optional

import zmq

from ..common.debug import flexkv_logger
from ..storage.gpu_layout import GpuRegistration, describe_gpu_tensors
from .request import GpuControlRequest, RegisterTPClientRequest, SlotMappingRequest
from .utils import get_zmq_socket


def registration_from_request(req: RegisterTPClientRequest) -> GpuRegistration:
    ptrs = [h.open() for h in req.handles]
    h0 = req.handles[0]
    if getattr(req, "is_swa", False):
        from ..storage.gpu_layout import swa_registration
        reg = swa_registration(ptrs, [h.shape for h in req.handles], [h.stride for h in req.handles], h0.dtype,
                               req.device_id if h0.device_id >= 0 else -1)
        reg.dp_client_id, reg.pp_rank, reg.tp_rank = req.dp_client_id, req.pp_rank, req.tp_rank
        reg.group_id = max(0, int(getattr(req, "group_id", 0)))
        reg.keepalive = list(req.handles)
        return reg
    reg = describe_gpu_tensors(ptrs, req.gpu_layout, h0.dtype, req.device_id if h0.device_id >= 0 else -1,
                               [h.shape for h in req.handles], [h.stride for h in req.handles])
    reg.dp_client_id, reg.pp_rank, reg.tp_rank = req.dp_client_id, req.pp_rank, req.tp_rank
    reg.group_id = getattr(req, "group_id", -1)
    reg.layer_groups = getattr(req, "layer_groups", None)
    reg.keepalive = list(req.handles)
    return reg


class RegistrationListener:
    def __init__(self, endpoint: str, on_register: Callable[[GpuRegistration], None],
                 on_control: Optional[Callable[[GpuControlRequest], bool]] = None,
                 on_slot_mapping: Optional[Callable[[SlotMappingRequest], None]] = None) -> None:
        self.endpoint = endpoint
        self.on_register = on_register
        self.on_control = on_control
        self.on_slot_mapping = on_slot_mapping
        self._ctx = zmq.Context.instance()
        self._sock = get_zmq_socket(self._ctx, zmq.PULL, endpoint, bind=True)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.count = 0

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, name="flexkv-gpu-register", daemon=True)
        self._thread.start()

    def _loop(self) -> None:
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        while not self._stop.is_set():
            if not dict(poller.poll(200)):
                continue
            try:
                req = pickle.loads(self._sock.recv())
                if isinstance(req, RegisterTPClientRequest):
                    self.on_register(registration_from_request(req))
                    self.count += 1
                    flexkv_logger.info("registered GPU tensors of dp client %d rank %d (device %d)",
                                       req.dp_client_id, req.intra_client_id, req.device_id)
                elif isinstance(req, SlotMappingRequest):
                    if self.on_slot_mapping is not None:
                        self.on_slot_mapping(req)
                elif isinstance(req, GpuControlRequest):
                    ok = False
                    try:
                        ok = bool(self.on_control(req)) if self.on_control is not None else False
                    finally:
                        if req.reply_endpoint:
                            rs = get_zmq_socket(self._ctx, zmq.PUSH, req.reply_endpoint, bind=False)
                            rs.send(pickle.dumps(ok))
                            rs.close(linger=1000)
            except Exception:  # noqa: BLE001
                flexkv_logger.exception("bad GPU registration message")

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        self._sock.close()
