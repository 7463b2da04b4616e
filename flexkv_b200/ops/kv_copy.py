"""Python entry points of the paged KV gather/scatter kernels.

``kv_copy`` launches on the caller's current CUDA stream and returns without
synchronising; block ids may be CUDA tensors, pinned host tensors or numpy
arrays (the latter are staged into a pinned buffer that the kernel reads in
place). There is no PyTorch fallback: on a machine with a GPU the native
module must be present.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import _native
from ..storage.gpu_layout import GpuRegistration

ENGINE_TMA = 0
ENGINE_SIMT = 1
STATUS_WORDS = 8


def new_status(device) -> torch.Tensor:
    """Status array for a launch: one int32 per error bit (see ``decode_status``)."""
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def decode_status(status: torch.Tensor) -> int:
    """Bit mask of the errors a launch reported (0 = clean): 1 GPU block id out of
    range, 2 host block id out of range, 4 a bounded wait expired, 8 bad arguments,
    16 payload overflow, 32 peer wait expired."""
    words = status.detach().cpu().tolist()
    return sum(1 << b for b, w in enumerate(words) if w)


@dataclass
class HostSide:
    base: int
    layer_stride: int
    kv_stride: int
    block_stride: int
    num_blocks: int
    offset: int = 0


def _ids_ptr(ids, keep: List[Any]) -> int:
    if isinstance(ids, torch.Tensor):
        if ids.dtype != torch.int64:
            raise TypeError("block ids must be int64")
        if not ids.is_cuda and not ids.is_pinned():
            ids = ids.pin_memory()
        keep.append(ids)
        return ids.data_ptr()
    t = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int64)).pin_memory()
    keep.append(t)
    return t.data_ptr()


def make_params(reg: GpuRegistration, host: HostSide, gpu_blocks, cpu_blocks, h2d: bool, layer_start: int = 0,
                num_layers: int = -1, chunk_bytes: Optional[int] = None, g_off: int = 0, status_ptr: int = 0,
                keep: Optional[List[Any]] = None) -> Dict[str, Any]:
    keep = keep if keep is not None else []
    n = int(len(gpu_blocks))
    if n != int(len(cpu_blocks)):
        raise ValueError("gpu and cpu block id lists differ in length")
    return dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul, idx_kv_mul=reg.idx_kv_mul,
                g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride, g_block_stride=reg.block_stride,
                g_off=g_off, cpu_base=int(host.base), c_layer_stride=host.layer_stride, c_kv_stride=host.kv_stride,
                c_block_stride=host.block_stride, c_off=host.offset, gpu_blocks_ptr=_ids_ptr(gpu_blocks, keep),
                cpu_blocks_ptr=_ids_ptr(cpu_blocks, keep), num_pairs=n, layer_start=layer_start,
                num_layers=reg.num_layers - layer_start if num_layers < 0 else num_layers, kv_dim=reg.kv_dim,
                chunk_bytes=reg.chunk_bytes if chunk_bytes is None else chunk_bytes,
                gpu_num_blocks=reg.num_blocks, cpu_num_blocks=host.num_blocks, status_ptr=status_ptr, h2d=int(h2d))


def kv_copy(reg: GpuRegistration, host: HostSide, gpu_blocks, cpu_blocks, h2d: bool, layer_start: int = 0,
            num_layers: int = -1, num_ctas: int = 16, tile_bytes: int = 16384, engine: int = ENGINE_TMA,
            status: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None,
            chunk_bytes: Optional[int] = None, g_off: int = 0) -> List[Any]:
    """Launches one gather/scatter. Returns objects that must stay alive until the
    stream has passed the launch (pinned id buffers)."""
    keep: List[Any] = []
    p = make_params(reg, host, gpu_blocks, cpu_blocks, h2d, layer_start, num_layers, chunk_bytes, g_off,
                    status.data_ptr() if status is not None else 0, keep)
    s = stream if stream is not None else torch.cuda.current_stream()
    _native.C.kv_copy(p, num_ctas, tile_bytes, engine, s.cuda_stream)
    return keep


def kv_copy_refshape(reg: GpuRegistration, host: HostSide, gpu_blocks, cpu_blocks, h2d: bool, num_ctas: int = 4,
                     stream: Optional[torch.cuda.Stream] = None) -> List[Any]:
    """Baseline launch shape (4 CTAs x 1024 threads, warp per chunk); timing comparisons only."""
    keep: List[Any] = []
    p = make_params(reg, host, gpu_blocks, cpu_blocks, h2d, keep=keep)
    s = stream if stream is not None else torch.cuda.current_stream()
    _native.C.kv_copy_refshape(p, num_ctas, s.cuda_stream)
    return keep


def host_kv_copy(reg: GpuRegistration, host: HostSide, gpu_blocks: np.ndarray, cpu_blocks: np.ndarray, h2d: bool,
                 layer_start: int = 0, num_layers: int = -1, threads: int = 4) -> int:
    """CPU oracle with identical addressing; every pointer is a host address."""
    g = np.ascontiguousarray(gpu_blocks, dtype=np.int64)
    c = np.ascontiguousarray(cpu_blocks, dtype=np.int64)
    p = dict(gpu_ptrs=[int(x) for x in reg.ptrs], idx_layer_mul=reg.idx_layer_mul, idx_kv_mul=reg.idx_kv_mul,
             g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride, g_block_stride=reg.block_stride,
             cpu_base=int(host.base), c_layer_stride=host.layer_stride, c_kv_stride=host.kv_stride,
             c_block_stride=host.block_stride, c_off=host.offset, gpu_blocks_ptr=g.ctypes.data,
             cpu_blocks_ptr=c.ctypes.data, num_pairs=int(g.size), layer_start=layer_start,
             num_layers=reg.num_layers - layer_start if num_layers < 0 else num_layers, kv_dim=reg.kv_dim,
             chunk_bytes=reg.chunk_bytes, gpu_num_blocks=reg.num_blocks, cpu_num_blocks=host.num_blocks,
             h2d=int(h2d))
    return _native.C.host_kv_copy(p, threads)
