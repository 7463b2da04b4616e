"""Small shared helpers."""
from __future__ import annotations

import contextlib
import os

try:  # NVTX ranges through torch's bundled bindings; a no-op when CUDA is absent
    import torch

    _NVTX = torch.cuda.nvtx if torch.cuda.is_available() and os.environ.get("FLEXKV_NVTX", "1") == "1" else None
except Exception:  # noqa: BLE001
    _NVTX = None


@contextlib.contextmanager
def nvtx_range(name: str):
    """Named range visible in Nsight timelines (reference marks the same phases:
    flexkv/kvtask.py:431,1066,1132; flexkv/transfer/transfer_engine.py:1151-1264)."""
    if _NVTX is None:
        yield
        return
    _NVTX.range_push(name)
    try:
        yield
    finally:
        _NVTX.range_pop()
