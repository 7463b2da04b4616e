"""NVSwitch fan-out restore (one process per GPU).

The ranks of a tensor-parallel group that hold identical KV (MLA latent cache)
allocate their paged caches out of one symmetric-memory buffer each, so that
the same byte offset in every rank's buffer is reachable through one multicast
address. A restore is then issued by ONE rank: its kernel reads each host block
over PCIe once and `multimem.st` writes it into every rank's cache; the other
ranks only wait for the completion flag in their signal area. The symmetric
allocation and rendezvous are torch.distributed plumbing; the data movement and
the flag are this package's kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .. import _native
from ..ops.kv_copy import HostSide, make_params
from ..storage.gpu_layout import GpuRegistration

FLAG_BYTES = 256      # tail of the symmetric buffer reserved for completion flags


@dataclass
class SymmetricKVBuffer:
    buffer: torch.Tensor          # uint8, symmetric
    handle: Any                   # torch symmetric-memory handle
    payload_bytes: int

    @property
    def local_ptr(self) -> int:
        return self.buffer.data_ptr()

    @property
    def multicast_ptr(self) -> int:
        return int(self.handle.multicast_ptr)

    @property
    def mc_delta(self) -> int:
        return self.multicast_ptr - self.local_ptr

    @property
    def flag_local_ptr(self) -> int:
        return self.local_ptr + self.payload_bytes

    @property
    def flag_mc_ptr(self) -> int:
        return self.multicast_ptr + self.payload_bytes

    def flag_tensor(self) -> torch.Tensor:
        return self.buffer[self.payload_bytes:self.payload_bytes + 4].view(torch.int32)

    def carve(self, offset: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        n = int(np.prod(shape)) * dtype.itemsize
        if offset % 256 or offset + n > self.payload_bytes:
            raise ValueError("carve out of range or misaligned")
        return self.buffer[offset:offset + n].view(dtype).view(*shape)


def alloc_symmetric_kv(payload_bytes: int, device: torch.device, group=None) -> SymmetricKVBuffer:
    """Collective: every rank of `group` allocates `payload_bytes` (+ flag area) of
    symmetric memory and exchanges handles. Raises if the fabric offers no multicast."""
    import torch.distributed._symmetric_memory as symm_mem
    group = group if group is not None else dist.group.WORLD
    payload_bytes = (payload_bytes + 255) // 256 * 256
    buf = symm_mem.empty(payload_bytes + FLAG_BYTES, dtype=torch.uint8, device=device)
    hdl = symm_mem.rendezvous(buf, group=group)
    if not int(getattr(hdl, "multicast_ptr", 0)):
        raise RuntimeError("symmetric memory has no multicast mapping on this system (NVLS unavailable)")
    buf.zero_()
    torch.cuda.synchronize(device)
    return SymmetricKVBuffer(buf, hdl, payload_bytes)


class SymmetricKVPool:
    """Several symmetric buffers used as one cache: every layer tensor lives entirely inside one segment and
    is reached through that segment's multicast mapping. Segments keep each multicast object small (the
    default is 2 GiB); the completion flags live in the tail of segment 0."""

    def __init__(self, segments: List[SymmetricKVBuffer], layers_per_segment: int, per_layer_bytes: int) -> None:
        self.segments = segments
        self.layers_per_segment = layers_per_segment
        self.per_layer_bytes = per_layer_bytes

    def layer_tensor(self, layer: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        seg = self.segments[layer // self.layers_per_segment]
        return seg.carve((layer % self.layers_per_segment) * self.per_layer_bytes, shape, dtype)

    def mc_of(self, ptr: int) -> int:
        """multicast address of a local address inside one of the segments"""
        for seg in self.segments:
            if seg.local_ptr <= ptr < seg.local_ptr + seg.payload_bytes:
                return ptr + seg.mc_delta
        raise ValueError("address outside the symmetric cache")

    # the flag area of segment 0 serves the whole pool
    @property
    def flag_mc_ptr(self) -> int:
        return self.segments[0].flag_mc_ptr

    def flag_tensor(self) -> torch.Tensor:
        return self.segments[0].flag_tensor()

    @property
    def mc_delta(self) -> int:
        return self.segments[0].mc_delta


def alloc_symmetric_kv_layers(num_layers: int, per_layer_bytes: int, device: torch.device, group=None,
                              segment_bytes: int = 2 << 30) -> SymmetricKVPool:
    """Collective: a symmetric cache of `num_layers` layers of `per_layer_bytes` each, in segments of at most
    `segment_bytes` (a whole number of layers per segment)."""
    per_layer_bytes = (per_layer_bytes + 255) // 256 * 256
    lps = max(1, min(num_layers, segment_bytes // per_layer_bytes))
    segs = []
    for l0 in range(0, num_layers, lps):
        segs.append(alloc_symmetric_kv(min(lps, num_layers - l0) * per_layer_bytes, device, group))
    return SymmetricKVPool(segs, lps, per_layer_bytes)


def fanout_restore(sym, reg: GpuRegistration, host: HostSide, gpu_blocks, cpu_blocks, epoch: int,
                   scratch: torch.Tensor, status: Optional[torch.Tensor] = None, layer_start: int = 0,
                   num_layers: int = -1, num_ctas: int = 8, tile_bytes: int = 16384,
                   stream: Optional[torch.cuda.Stream] = None) -> List[Any]:
    """Issuing rank only: host blocks -> every rank's cache, then flag := epoch on
    every rank. `sym` is a SymmetricKVBuffer or a SymmetricKVPool; `scratch` is a zeroed int32
    device word reused across calls."""
    keep: List[Any] = []
    p = make_params(reg, host, gpu_blocks, cpu_blocks, True, layer_start, num_layers,
                    status_ptr=status.data_ptr() if status is not None else 0, keep=keep)
    p["done_counter_ptr"] = scratch.data_ptr()
    p["epoch"] = int(epoch)
    if isinstance(sym, SymmetricKVPool):
        p["mc_ptrs"] = [sym.mc_of(int(a)) for a in reg.ptrs]
    s = stream if stream is not None else torch.cuda.current_stream()
    _native.C.kv_fanout(p, sym.mc_delta, sym.flag_mc_ptr, num_ctas, tile_bytes, s.cuda_stream)
    return keep


def wait_flag(sym, epoch: int, timeout_s: float = 10.0) -> bool:
    """Receiving ranks: host-side bounded wait for the completion flag."""
    import time
    flag = sym.flag_tensor()
    t0 = time.monotonic()
    while time.monotonic() - t0 < timeout_s:
        if int(flag.item()) - epoch >= 0:
            return True
        time.sleep(0.0002)
    return False
