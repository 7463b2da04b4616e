"""ZeroMQ socket helpers (flexkv/server/utils.py:5-41)."""
from __future__ import annotations

import os
import tempfile
import uuid

import zmq


def get_zmq_socket(ctx: zmq.Context, sock_type: int, endpoint: str, bind: bool) -> zmq.Socket:
    s = ctx.socket(sock_type)
    s.setsockopt(zmq.LINGER, 0)
    if sock_type in (zmq.PUSH, zmq.PULL):
        s.setsockopt(zmq.SNDHWM, 0)
        s.setsockopt(zmq.RCVHWM, 0)
    if bind:
        if endpoint.startswith("ipc://"):
            path = endpoint[len("ipc://"):]
            if os.path.exists(path):
                os.unlink(path)
        s.bind(endpoint)
    else:
        s.connect(endpoint)
    return s


def unique_ipc_endpoint(prefix: str = "flexkv") -> str:
    return f"ipc://{tempfile.gettempdir()}/{prefix}_{os.getpid()}_{uuid.uuid4().hex[:8]}"
