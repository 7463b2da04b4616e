"""Lossless exponent-packing codec for bf16 KV (see csrc/kernels/kv_compress.h for
the format) — launcher and a bit-exact PyTorch reference of the packed bytes."""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from .. import _native
from ..storage.gpu_layout import GpuRegistration
from .kv_copy import HostSide, make_params

TILE_ELEMS = 8192
TILE_SLOT = 2 * TILE_ELEMS + 128
GROUP = 128


def tiles_per_chunk(chunk_elems: int) -> int:
    return (chunk_elems + TILE_ELEMS - 1) // TILE_ELEMS


def chunk_slot_bytes(chunk_elems: int) -> int:
    return tiles_per_chunk(chunk_elems) * TILE_SLOT


def size_table_entries(num_blocks: int, num_layers: int, kv_dim: int, chunk_elems: int) -> int:
    return num_blocks * num_layers * kv_dim * tiles_per_chunk(chunk_elems)


def kv_compress(reg: GpuRegistration, host: HostSide, size_table: torch.Tensor, gpu_blocks, cpu_blocks, h2d: bool,
                layers_total: Optional[int] = None, layer_start: int = 0, num_layers: int = -1, num_ctas: int = 32,
                status: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> List[Any]:
    """compress (GPU -> host, ``h2d=False``) or decompress on the current stream.
    ``size_table`` is a pinned uint32/int32 tensor the kernel addresses directly."""
    if reg.dtype != torch.bfloat16:
        raise TypeError("the exponent-packing codec serves bf16 caches")
    keep: List[Any] = []
    p = make_params(reg, host, gpu_blocks, cpu_blocks, h2d, layer_start, num_layers,
                    status_ptr=status.data_ptr() if status is not None else 0, keep=keep)
    s = stream if stream is not None else torch.cuda.current_stream()
    _native.C.kv_compress_bf16(p, size_table.data_ptr(), layers_total or reg.num_layers, num_ctas, s.cuda_stream)
    return keep


def reference_compress_tile(x: torch.Tensor) -> torch.Tensor:
    """Packed bytes (uint8, 1-D) of one tile of bf16 values (numel % 1024 == 0, <= 8192)."""
    v = x.reshape(-1).view(torch.int16).to(torch.int32) & 0xFFFF
    G = v.numel() // GROUP
    v = v.reshape(G, GROUP)
    e = (v >> 7) & 0xFF
    emax, emin = e.amax(1), e.amin(1)
    rng = (emax - emin)
    w = torch.where(rng == 0, torch.zeros_like(rng), torch.floor(torch.log2(rng.clamp(min=1).float())).int() + 1)
    hdr = torch.stack([emax, w], 1).to(torch.uint8).reshape(-1)
    smb = (((v >> 8) & 0x80) | (v & 0x7F)).to(torch.uint8)
    d = emax[:, None] - e                                  # [G, 128]; element index = 4*lane + j
    d = d.reshape(G, 32, 4)
    lanes = torch.arange(32, dtype=torch.int64)
    out = [hdr]
    for g in range(G):
        out.append(smb[g])
        for b in range(int(w[g])):
            for j in range(4):
                bits = ((d[g, :, j] >> b) & 1).to(torch.int64)
                word = int((bits << lanes).sum().item()) & 0xFFFFFFFF
                out.append(torch.tensor([word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF, (word >> 24) & 0xFF],
                                        dtype=torch.uint8))
    return torch.cat(out)
