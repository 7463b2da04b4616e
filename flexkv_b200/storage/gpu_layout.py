"""Addressing of an engine's registered paged KV tensors.

The number of tensors a rank registers selects the addressing rule, as in the
reference (csrc/tp_transfer_thread_group.cpp:71-80, csrc/gtensor_handler.cuh:43-67):

* ``num_layers`` tensors  -> vLLM: one tensor per layer, ``[2, N, T, H, D]``
  (LAYERFIRST), ``[N, 2, T, H, D]`` (LAYERBLOCK) or MLA ``[N, T, D]``;
* ``2 * num_layers``      -> SGLang: all K buffers, then all V buffers;
* ``1``                   -> TensorRT-LLM: one tensor ``[N, L, kv, ...]``.

The strides are taken from the layout the engine declares and checked against
the real tensors where the tensors are visible (flexkv/transfer/worker.py:262-306).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..common.storage import KVCacheLayout, KVCacheLayoutType


@dataclass
class GpuRegistration:
    """Everything the data plane needs to address one rank's KV cache."""
    device_id: int
    ptrs: List[int]
    backend: str                    # vllm | sglang | trtllm
    idx_layer_mul: int
    idx_kv_mul: int
    layer_stride: int               # bytes
    kv_stride: int
    block_stride: int
    chunk_bytes: int
    num_blocks: int
    num_layers: int
    kv_dim: int
    dtype: torch.dtype
    dp_client_id: int = 0
    pp_rank: int = 0
    tp_rank: int = 0                # effective rank inside the host block (cp_rank * tp + tp_rank)
    group_id: int = -1              # layer group of a multi-group cache (-1: the only group)
    is_swa: bool = False            # sliding-window pages (group_id then names the window pool's group)
    layer_groups: Any = None        # LayerGroupSpec list sent along by a worker that discovered the groups itself
    # NVSwitch multicast: mc_ptrs[i] is the multicast address of tensor ptrs[i] (one store there lands in every
    # rank's copy of the tensor), mc_flag_ptr the multicast address of the ranks' completion flag. A registration
    # that carries them stands for all ranks of its shared-KV tensor-parallel group.
    mc_ptrs: Optional[List[int]] = None
    mc_flag_ptr: int = 0
    keepalive: Any = field(default=None, repr=False)   # tensors or opened handles

    def as_native(self) -> Dict[str, Any]:
        return dict(device=self.device_id, ptrs=[int(p) for p in self.ptrs], idx_layer_mul=self.idx_layer_mul,
                    idx_kv_mul=self.idx_kv_mul, layer_stride=self.layer_stride, kv_stride=self.kv_stride,
                    block_stride=self.block_stride, num_blocks=self.num_blocks)


def describe_gpu_tensors(ptrs: Sequence[int], gpu_layout: KVCacheLayout, dtype: torch.dtype, device_id: int,
                         tensor_shapes: Optional[Sequence[Sequence[int]]] = None,
                         tensor_strides: Optional[Sequence[Sequence[int]]] = None) -> GpuRegistration:
    L, K = gpu_layout.num_layer, gpu_layout.kv_dim
    isz = dtype.itemsize
    chunk = gpu_layout.get_chunk_size() * isz
    n = len(ptrs)
    if n == L and not (L == 1 and gpu_layout.type == KVCacheLayoutType.BLOCKFIRST):
        backend = "vllm"
        per_layer = gpu_layout._replace(num_layer=1)
        if gpu_layout.type == KVCacheLayoutType.BLOCKFIRST:
            raise ValueError("a per-layer registration cannot be BLOCKFIRST")
        kv_stride = per_layer.get_kv_stride() * isz
        block_stride = per_layer.get_block_stride() * isz
        reg = GpuRegistration(device_id, list(ptrs), backend, 1, 0, 0, kv_stride, block_stride, chunk,
                              gpu_layout.num_block, L, K, dtype)
    elif n == 2 * L and K == 2:
        backend = "sglang"
        reg = GpuRegistration(device_id, list(ptrs), backend, 1, L, 0, 0, chunk, chunk, gpu_layout.num_block, L, K,
                              dtype)
    elif n == 1:
        backend = "trtllm"
        if gpu_layout.type == KVCacheLayoutType.BLOCKFIRST:
            ls, ks, bs = gpu_layout.get_layer_stride(), gpu_layout.get_kv_stride(), gpu_layout.get_block_stride()
        else:
            ls, ks, bs = gpu_layout.get_layer_stride(), gpu_layout.get_kv_stride(), gpu_layout.get_block_stride()
        reg = GpuRegistration(device_id, list(ptrs), backend, 0, 0, ls * isz, ks * isz, bs * isz, chunk,
                              gpu_layout.num_block, L, K, dtype)
    else:
        raise ValueError(f"cannot infer the engine layout from {n} tensors for {L} layers (kv_dim {K})")
    if tensor_shapes is not None and tensor_strides is not None:
        _check_against_tensors(reg, tensor_shapes, tensor_strides, isz)
    return reg


def _check_against_tensors(reg: GpuRegistration, shapes, strides, isz: int) -> None:
    """Every registered tensor must be dense and large enough for the declared block count."""
    per_tensor_bytes = {
        "vllm": reg.kv_dim * reg.num_blocks * reg.chunk_bytes,
        "sglang": reg.num_blocks * reg.chunk_bytes,
        "trtllm": reg.num_blocks * reg.block_stride,
    }[reg.backend]
    for shp, st in zip(shapes, strides):
        numel = 1
        for d in shp:
            numel *= int(d)
        if numel * isz < per_tensor_bytes:
            raise ValueError(f"registered tensor of {numel * isz} bytes is smaller than the declared layout "
                             f"({per_tensor_bytes} bytes)")
        expect = 1
        for d, s in zip(reversed(list(shp)), reversed(list(st))):
            if int(d) != 1 and int(s) != expect:
                raise ValueError("registered KV tensors must be contiguous")
            expect *= int(d)


def register_tensors(tensors: Sequence[torch.Tensor], gpu_layout: KVCacheLayout, **ids) -> GpuRegistration:
    dev = (tensors[0].device.index or 0) if tensors[0].is_cuda else -1   # -1: host-resident stand-in
    reg = describe_gpu_tensors([t.data_ptr() for t in tensors], gpu_layout, tensors[0].dtype, dev,
                               [tuple(t.shape) for t in tensors], [tuple(t.stride()) for t in tensors])
    reg.keepalive = list(tensors)
    for k, v in ids.items():
        setattr(reg, k, v)
    return reg


def swa_registration(ptrs: Sequence[int], shapes: Sequence[Sequence[int]], strides: Sequence[Sequence[int]],
                     dtype: torch.dtype, device_id: int) -> GpuRegistration:
    """Window pages of one rank: one tensor per layer, ``[num_pages, ...]`` with a contiguous page."""
    s0 = tuple(int(d) for d in shapes[0])
    page_elems = 1
    for d in s0[1:]:
        page_elems *= d
    for shp, st in zip(shapes, strides):
        expect = 1
        for d, s in zip(reversed(list(shp)), reversed(list(st))):
            if int(d) != 1 and int(s) != expect:
                raise ValueError("window page tensors must be contiguous")
            expect *= int(d)
        if tuple(int(d) for d in shp) != s0:
            raise ValueError("window page tensors must be identically shaped")
    page_bytes = page_elems * dtype.itemsize
    return GpuRegistration(device_id, [int(p) for p in ptrs], "vllm", 1, 0, 0, 0, page_bytes, page_bytes, s0[0],
                           len(ptrs), 1, dtype, is_swa=True)
