"""Stand-alone KV server: ``python -m flexkv_b200.server --model-config m.json --cache-config c.json
--recv-endpoint ipc:///tmp/flexkv_server --gpu-register-port ipc:///tmp/flexkv_gpu``.

Engine instances then run with ``FLEXKV_SERVER_LAUNCH_MODE=external`` and the same endpoints: their
``KVManager`` only creates clients, and their workers register tensors through ``KVTPClient``
(external server mode of the reference: flexkv/server/server.py:299-345, tests/test_external_server_mode.py).
The JSON files hold the fields of ``ModelConfig`` / ``CacheConfig``; ``dtype`` is a torch dtype name.
"""
from __future__ import annotations

import argparse
import json
import signal

from ..common.config import CacheConfig, ModelConfig, parse_dtype
from ..common.debug import flexkv_logger
from .server import KVServer


def _load(path_or_json: str) -> dict:
    s = path_or_json.strip()
    if s.startswith("{"):
        return json.loads(s)
    with open(s) as f:
        return json.load(f)


def main() -> None:
    ap = argparse.ArgumentParser(description="flexkv_b200 KV server")
    ap.add_argument("--model-config", required=True, help="JSON file or inline JSON with ModelConfig fields")
    ap.add_argument("--cache-config", required=True, help="JSON file or inline JSON with CacheConfig fields")
    ap.add_argument("--recv-endpoint", required=True)
    ap.add_argument("--gpu-register-port", required=True)
    ap.add_argument("--no-gpu", action="store_true", help="serve host-resident stand-in tensors (tests)")
    a = ap.parse_args()
    m = _load(a.model_config)
    if "dtype" in m:
        m["dtype"] = parse_dtype(m["dtype"])
    model = ModelConfig(**m)
    cache = CacheConfig(**_load(a.cache_config))
    srv = KVServer(model, cache, a.recv_endpoint, a.gpu_register_port, require_gpu=True if a.no_gpu else None)
    signal.signal(signal.SIGINT, signal.SIG_IGN)
    signal.signal(signal.SIGTERM, lambda *_: setattr(srv, "_running", False))
    flexkv_logger.info("KV server listening on %s (GPU registrations on %s)", a.recv_endpoint, a.gpu_register_port)
    try:
        srv.run()
    finally:
        srv.engine.shutdown()


if __name__ == "__main__":
    main()
