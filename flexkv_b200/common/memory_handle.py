"""Handles that let another process address a tensor.

``TensorSharedHandle`` describes one KV tensor of an engine worker: device,
dtype, shape, strides and how to reach its memory. Two modes:

* ``same_process`` — producer and consumer share the address space; the handle
  carries the address and a registry keeps the tensor alive;
* ``cuda_ipc`` — a CUDA IPC handle of the tensor's allocation plus the tensor's
  offset inside it; the importer opens the allocation on its own context.

The reference also offers VMM fabric / POSIX-fd exports for allocations made
with the virtual-memory API (flexkv/common/memory_handle.py:466-545,1144-1250);
they apply to engines that allocate their cache with cuMemCreate and are not
needed for torch-allocated caches.
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native

_registry: Dict[int, Any] = {}
_registry_lock = threading.Lock()
_opened: Dict[Tuple[bytes, int], Tuple[int, int]] = {}     # (handle, device) -> (base address, refcount)


@dataclass
class TensorSharedHandle:
    mode: str
    device_id: int
    dtype: torch.dtype
    shape: Tuple[int, ...]
    stride: Tuple[int, ...]
    nbytes: int
    pid: int
    address: int = 0                      # same_process
    ipc_handle: bytes = b""               # cuda_ipc
    ipc_offset: int = 0
    _base: int = field(default=0, repr=False, compare=False)

    @classmethod
    def export(cls, t: torch.Tensor, mode: Optional[str] = None, same_process_ok: bool = True) -> "TensorSharedHandle":
        if not t.is_contiguous():
            raise ValueError("only contiguous tensors can be shared")
        dev = t.device.index if t.is_cuda else -1
        common = dict(device_id=dev if dev is not None else 0, dtype=t.dtype, shape=tuple(t.shape),
                      stride=tuple(t.stride()), nbytes=t.numel() * t.element_size(), pid=os.getpid())
        if mode is None:
            mode = "cuda_ipc" if t.is_cuda else "same_process"
        if mode == "same_process" or not t.is_cuda:
            with _registry_lock:
                _registry[t.data_ptr()] = t
            return cls(mode="same_process", address=t.data_ptr(), **common)
        if mode != "cuda_ipc":
            raise ValueError(f"unsupported handle mode {mode}")
        handle, offset, _ = _native.C.ipc_export(t.data_ptr())
        with _registry_lock:
            _registry[t.data_ptr()] = t       # the exporter must outlive the importer's mapping
        return cls(mode="cuda_ipc", ipc_handle=bytes(handle), ipc_offset=int(offset), address=t.data_ptr(), **common)

    def open(self) -> int:
        """Device address of the tensor in this process."""
        if self.mode == "same_process" or self.pid == os.getpid():
            return self.address
        key = (self.ipc_handle, self.device_id)
        with _registry_lock:
            if key in _opened:
                base, n = _opened[key]
                _opened[key] = (base, n + 1)
            else:
                base = _native.C.ipc_import(self.ipc_handle, self.device_id)
                _opened[key] = (base, 1)
        self._base = base
        return base + self.ipc_offset

    def close(self) -> None:
        if self.mode != "cuda_ipc" or self.pid == os.getpid() or not self._base:
            return
        key = (self.ipc_handle, self.device_id)
        with _registry_lock:
            base, n = _opened.get(key, (0, 0))
            if n <= 1:
                _opened.pop(key, None)
                if base:
                    _native.C.ipc_close(base, self.device_id)
            else:
                _opened[key] = (base, n - 1)
        self._base = 0

    def __getstate__(self):
        d = dict(self.__dict__)
        d["_base"] = 0
        d["dtype"] = str(self.dtype).replace("torch.", "")
        return d

    def __setstate__(self, d):
        d = dict(d)
        d["dtype"] = getattr(torch, d["dtype"])
        self.__dict__.update(d)


def release_exported(t: torch.Tensor) -> None:
    with _registry_lock:
        _registry.pop(t.data_ptr(), None)
