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

* ``vmm_fabric`` / ``vmm_posix_fd`` — memory that an engine allocated with the virtual-memory
  API (cuMemCreate + cuMemMap, e.g. a sleep-mode allocator) has no legacy IPC handle. The
  physical allocation is exported as a fabric handle (64 bytes inside the pickled handle)
  where the allocation allows it, else as a POSIX file descriptor that the importer fetches
  from the exporter's descriptor server (a UNIX socket, SCM_RIGHTS); the importer maps it
  into an address range of its own (flexkv/common/memory_handle.py:466-545,600-700,800-900).
  ``export`` picks these modes by itself when the tensor's memory is a cuMemCreate mapping.
"""
from __future__ import annotations

import array
import os
import socket
import struct
import tempfile
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native

_registry: Dict[int, Any] = {}
_registry_lock = threading.Lock()
_opened: Dict[Tuple[bytes, int], Tuple[int, int]] = {}     # (handle, device) -> (base address, refcount)
_vmm_opened: Dict[Tuple[int, int, int], List[int]] = {}    # (exporter pid, exporter base, device) -> [va, size, refs]


# ---- descriptor server of the exporting process ---------------------------------------------
# One daemon thread per process serves the descriptors of its exported allocations: a client
# sends the 8-byte token it found in the handle and receives a duplicate through SCM_RIGHTS.
_fd_exports: Dict[int, int] = {}          # token -> descriptor (stays open while the export lives)
_fd_server: Optional[socket.socket] = None
_fd_server_path = ""


def fd_server_path(pid: int) -> str:
    return os.path.join(os.environ.get("FLEXKV_VMM_FD_DIR") or os.environ.get("FLEXKV_VMM_FD_SOCK_DIR") or tempfile.gettempdir(), f"flexkv_vmm_fd_{pid}.sock")


def _serve_fds(srv: socket.socket) -> None:
    while True:
        try:
            conn, _ = srv.accept()
        except OSError:
            return                               # socket closed
        with conn:
            try:
                conn.settimeout(5.0)
                raw = b""
                while len(raw) < 8:
                    part = conn.recv(8 - len(raw))
                    if not part:
                        break
                    raw += part
                if len(raw) < 8:
                    continue
                (token,) = struct.unpack("q", raw)
                with _registry_lock:
                    fd = _fd_exports.get(token)
                if fd is None:
                    conn.sendall(b"\0")          # unknown token: one byte, no descriptor
                else:
                    conn.sendmsg([b"\1"], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))])
            except OSError:
                continue


def serve_fd(fd: int) -> Tuple[int, str]:
    """Registers ``fd`` with this process's descriptor server (started on first use) and returns
    ``(token, socket path)`` for the handle."""
    global _fd_server, _fd_server_path
    with _registry_lock:
        if _fd_server is None:
            path = fd_server_path(os.getpid())
            if os.path.exists(path):
                os.unlink(path)
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            srv.bind(path)
            srv.listen(64)
            _fd_server, _fd_server_path = srv, path
            threading.Thread(target=_serve_fds, args=(srv,), name="flexkv-vmm-fd-server", daemon=True).start()
        _fd_exports[int(fd)] = int(fd)
        return int(fd), _fd_server_path


def fetch_fd(sock_path: str, token: int, timeout: float = 10.0) -> int:
    """Importer side: a duplicate of the exporter's descriptor ``token``."""
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
        s.settimeout(timeout)
        s.connect(sock_path)
        s.sendall(struct.pack("q", int(token)))
        fds = array.array("i")
        msg, anc, _, _ = s.recvmsg(1, socket.CMSG_LEN(fds.itemsize))
        for level, ctype, data in anc:
            if level == socket.SOL_SOCKET and ctype == socket.SCM_RIGHTS:
                fds.frombytes(data[:len(data) - (len(data) % fds.itemsize)])
        if msg != b"\1" or len(fds) != 1:
            for fd in fds:
                os.close(fd)
            raise RuntimeError(f"the exporter at {sock_path} does not serve descriptor {token}")
        return int(fds[0])


def stop_fd_server() -> None:
    global _fd_server, _fd_server_path
    with _registry_lock:
        srv, path = _fd_server, _fd_server_path
        _fd_server, _fd_server_path = None, ""
        fds = list(_fd_exports.values())
        _fd_exports.clear()
    if srv is not None:
        srv.close()
        try:
            os.unlink(path)
        except OSError:
            pass
    for fd in fds:
        try:
            os.close(fd)
        except OSError:
            pass


_vmm_exports: Dict[int, Dict[str, Any]] = {}       # exporter's range base -> handle fields shared by its tensors


def _export_vmm(ptr: int, mode: str) -> Dict[str, Any]:
    """Handle fields for a pointer inside a cuMemCreate mapping. Tensors carved out of one
    allocation share one export (one descriptor or fabric handle per allocation)."""
    e = _native.C.vmm_export(ptr, mode != "vmm_posix_fd")
    base = int(e["base"])
    with _registry_lock:
        known = _vmm_exports.get(base)
    if known is not None and (mode == "vmm" or known["mode"] == mode):
        if e["kind"] == "posix_fd":
            os.close(int(e["fd"]))                   # the first export's descriptor is the one served
        return dict(known, vmm_offset=int(e["offset"]), address=ptr)
    fields: Dict[str, Any] = dict(vmm_base=base, vmm_size=int(e["size"]))
    if e["kind"] == "fabric":
        fields.update(mode="vmm_fabric", vmm_fabric=bytes(e["fabric"]))
    elif mode == "vmm_fabric":
        os.close(int(e["fd"]))
        raise ValueError("the allocation cannot be exported as a fabric handle")
    else:
        token, path = serve_fd(int(e["fd"]))
        fields.update(mode="vmm_posix_fd", vmm_fd_token=token, vmm_fd_socket=path)
    with _registry_lock:
        _vmm_exports[base] = dict(fields)
    return dict(fields, vmm_offset=int(e["offset"]), address=ptr)


class DeviceSpan:
    """A raw device range as an object torch can wrap: ``torch.as_tensor(DeviceSpan(...), device=...)``."""

    def __init__(self, address: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(address), False),
                                         "version": 2, "strides": None}


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
    vmm_fabric: bytes = b""               # vmm_fabric
    vmm_fd_token: int = -1                # vmm_posix_fd: token at the exporter's descriptor server
    vmm_fd_socket: str = ""
    vmm_base: int = 0                     # exporter's mapped range that holds the tensor
    vmm_size: int = 0
    vmm_offset: int = 0
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
            if t.is_cuda and _native.C.vmm_is_vmm_pointer(t.data_ptr()):
                mode = "vmm"                      # fabric where the allocation allows it, else a descriptor
        if mode == "host_file":
            if shared_file is None:
                raise ValueError("host_file handles need a tensor from alloc_shared_host_tensor")
            path, base = shared_file
            return cls(mode="host_file", address=t.data_ptr(), file_path=path, file_offset=t.data_ptr() - base, **common)
        if mode == "same_process" or not t.is_cuda:
            with _registry_lock:
                _registry[t.data_ptr()] = t
            return cls(mode="same_process", address=t.data_ptr(), **common)
        if mode in ("vmm", "vmm_fabric", "vmm_posix_fd"):
            with _registry_lock:
                _registry[t.data_ptr()] = t
            return cls(**_export_vmm(t.data_ptr(), mode), **common)
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
        if self.mode in ("vmm_fabric", "vmm_posix_fd"):
            key3 = (self.pid, self.vmm_base, self.device_id)
            with _registry_lock:
                ent = _vmm_opened.get(key3)
                if ent is not None:
                    ent[2] += 1
                else:
                    if self.mode == "vmm_fabric":
                        va, size = _native.C.vmm_import_fabric(self.vmm_fabric, self.vmm_size, self.device_id)
                    else:
                        fd = fetch_fd(self.vmm_fd_socket, self.vmm_fd_token)
                        try:
                            va, size = _native.C.vmm_import_fd(fd, self.vmm_size, self.device_id)
                        finally:
                            os.close(fd)            # the mapping keeps the memory; the duplicate is done
                    ent = _vmm_opened[key3] = [int(va), int(size), 1]
            self._base = ent[0]
            return ent[0] + self.vmm_offset
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
        if self.mode in ("vmm_fabric", "vmm_posix_fd") and self.pid != os.getpid() and self._base:
            key3 = (self.pid, self.vmm_base, self.device_id)
            with _registry_lock:
                ent = _vmm_opened.get(key3)
                if ent is not None:
                    ent[2] -= 1
                    if ent[2] <= 0:
                        _vmm_opened.pop(key3, None)
                        _native.C.vmm_unmap(ent[0], ent[1])
            self._base = 0
            return
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
