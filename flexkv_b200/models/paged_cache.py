"""Synthetic paged KV caches in the three engine layouts.

* ``vllm``   : one tensor per layer, ``[2, N, T, H, D]`` (or ``[N, T, D]`` for MLA,
               ``[N, 2, T, H, D]`` with ``layerblock=True``)
* ``sglang`` : ``2L`` tensors, all K buffers then all V buffers, each ``[N, T, H, D]``
* ``trtllm`` : one tensor ``[N, L, kv, T, H, D]``
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from ..common.storage import KVCacheLayout, KVCacheLayoutType
from .shapes import KVShape


def alloc_paged_cache(shape: KVShape, num_blocks: int, device, engine_layout: str = None, tp_size: int = 1,
                      layerblock: bool = False, fill: str = "zeros", seed: int = 0
                      ) -> Tuple[List[torch.Tensor], KVCacheLayout]:
    engine_layout = engine_layout or shape.engine_layout
    L, T, D = shape.num_layers, shape.tokens_per_block, shape.head_size
    H = shape.num_kv_heads if shape.use_mla else max(1, shape.num_kv_heads // tp_size)
    K = shape.kv_dim
    N = num_blocks
    dt = shape.dtype

    def new(*dims):
        return torch.empty(*dims, dtype=dt, device=device)

    if engine_layout == "vllm":
        if shape.use_mla:
            tensors = [new(N, T, H * D) for _ in range(L)]
            ltype = KVCacheLayoutType.LAYERFIRST
        elif layerblock:
            tensors = [new(N, 2, T, H, D) for _ in range(L)]
            ltype = KVCacheLayoutType.LAYERBLOCK
        else:
            tensors = [new(2, N, T, H, D) for _ in range(L)]
            ltype = KVCacheLayoutType.LAYERFIRST
    elif engine_layout == "sglang":
        if K != 2:
            tensors = [new(N, T, H * D) for _ in range(L)]
        else:
            tensors = [new(N, T, H, D) for _ in range(2 * L)]
        ltype = KVCacheLayoutType.LAYERFIRST
    elif engine_layout == "trtllm":
        tensors = [new(N, L, K, T, H, D)]
        ltype = KVCacheLayoutType.BLOCKFIRST
    else:
        raise ValueError(f"unknown engine layout {engine_layout}")
    layout = KVCacheLayout(ltype, L, N, T, H, D, is_mla=shape.use_mla, kv_dim_override=K)
    fill_cache(tensors, fill, seed)
    return tensors, layout


def fill_cache(tensors: List[torch.Tensor], fill: str, seed: int = 0) -> None:
    if fill == "zeros":
        for t in tensors:
            t.zero_()
        return
    g = torch.Generator(device=tensors[0].device)
    g.manual_seed(seed)
    for t in tensors:
        flat = t.view(-1)
        step = 1 << 28
        for lo in range(0, flat.numel(), step):
            part = flat[lo:lo + step]
            if t.dtype == torch.uint8:
                part.copy_(torch.randint(0, 256, part.shape, generator=g, device=t.device, dtype=torch.uint8))
            elif fill == "normal":
                part.copy_(torch.randn(part.shape, generator=g, device=t.device, dtype=torch.float32).to(t.dtype))
            else:
                raise ValueError(f"unknown fill {fill}")
