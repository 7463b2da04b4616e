"""Handles that let another process address a tensor.

``TensorSharedHandle`` describes one KV tensor of an engine worker: device,
dtype, shape, strides and how to reach its memory. Two modes:

* ``same_process`` — producer and consumer share the address space; the handle
  carries the address and a registry keeps the tensor alive;
* ``cuda_ipc`` — a CUDA IPC handle of the tensor's allocation plus the tensor's
  offset inside it; the importer opens the allocation on its own context;
* ``host_file`` — a host tensor that lives in a shared file (``alloc_shared_host_tensor``);
  the importer maps the same file. Used by GPU-less deployments and tests whose "GPU"
  tensors are host stand-ins owned by another process.

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
    file_path: str = ""                   # host_file
    file_offset: int = 0
    _base: int = field(default=0, repr=False, compare=False)

    @classmethod
    def export(cls, t: torch.Tensor, mode: Optional[str] = None, same_process_ok: bool = True) -> "TensorSharedHandle":
        if not t.is_contiguous():
            raise ValueError("only contiguous tensors can be shared")
        dev = t.device.index if t.is_cuda else -1
        common = dict(device_id=dev if dev is not None else 0, dtype=t.dtype, shape=tuple(t.shape),
                      stride=tuple(t.stride()), nbytes=t.numel() * t.element_size(), pid=os.getpid())
        shared_file = _shared_files.get(t.untyped_storage().data_ptr()) if not t.is_cuda else None
        if mode is None:
            mode = "cuda_ipc" if t.is_cuda else ("host_file" if shared_file is not None else "same_process")
        if mode == "host_file":
            if shared_file is None:
                raise ValueError("host_file handles need a tensor from alloc_shared_host_tensor")
            path, base = shared_file
            return cls(mode="host_file", address=t.data_ptr(), file_path=path, file_offset=t.data_ptr() - base, **common)
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
        if self.mode == "host_file":
            import numpy as np
            with _registry_lock:
                mm = _mapped_files.get(self.file_path)
                if mm is None:
                    mm = np.memmap(self.file_path, dtype=np.uint8, mode="r+")
                    _mapped_files[self.file_path] = mm
            return int(mm.ctypes.data) + self.file_offset
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


_shared_files: Dict[int, Tuple[str, int]] = {}      # storage address -> (file, base address)
_mapped_files: Dict[str, Any] = {}


def alloc_shared_host_tensor(shape: Sequence[int], dtype: torch.dtype, path: str) -> torch.Tensor:
    """A host tensor backed by ``path`` (e.g. under /dev/shm) that other processes can open
    through a ``host_file`` handle."""
    n = 1
    for d in shape:
        n *= int(d)
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    with open(path, "wb") as f:
        f.truncate(nbytes)
    flat = torch.from_file(path, shared=True, size=nbytes, dtype=torch.uint8)
    with _registry_lock:
        _shared_files[flat.untyped_storage().data_ptr()] = (path, flat.data_ptr())
    return flat.view(dtype).view(*shape)


def release_exported(t: torch.Tensor) -> None:
    with _registry_lock:
        _registry.pop(t.data_ptr(), None)
