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
    # full tiles take a full slot; the last, shorter tile takes what its own raw form would need
    full, rest = divmod(chunk_elems, TILE_ELEMS)
    return full * TILE_SLOT + ((2 * rest + 128) if rest else 0)


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


CHUNK_VALS = 64
HEADER_BYTES = 32
RANKS, SHORT_RANKS, ESCAPE_ONES = 16, 3, 13
FLAT_ESCAPE_ONES = 4
SAMPLE_WORDS = 4
SAMPLE_STRIDE = CHUNK_VALS // 2 // SAMPLE_WORDS      # words 0, 8, 16, 24 of every chunk are sampled


def _code_of(rank: int, exponent: int, mode: int = 1):
    """(bits, length) of one exponent, LSB first; rank >= RANKS means no code of its own."""
    if mode == 2:
        if rank < RANKS:
            q = rank >> 2
            return ((1 << q) - 1) | ((rank & 3) << (q + 1)), q + 3
        return ((1 << FLAT_ESCAPE_ONES) - 1) | (exponent << FLAT_ESCAPE_ONES), FLAT_ESCAPE_ONES + 8
    if rank < SHORT_RANKS:
        return rank, 2
    if rank < RANKS:
        n = rank - SHORT_RANKS
        return 3 | (((1 << n) - 1) << 2), n + 3
    return 3 | (((1 << ESCAPE_ONES) - 1) << 2) | (exponent << (2 + ESCAPE_ONES)), 2 + ESCAPE_ONES + 8


def reference_compress_tile(x: torch.Tensor) -> torch.Tensor:
    """Packed bytes (uint8, 1-D) of one tile of bf16 values (numel % 1024 == 0, <= 8192), computed on the
    CPU with plain Python integers from the format description alone."""
    import numpy as np
    v = x.reshape(-1).view(torch.int16).numpy().view(np.uint16).astype(np.int64)
    n = v.size
    C = n // CHUNK_VALS
    e = (v >> 7) & 0xFF
    # frequencies over the sample the format names: every SAMPLE_STRIDE-th word of every chunk
    sample = [2 * (k * C + t) + h for t in range(C) for k in range(0, CHUNK_VALS // 2, SAMPLE_STRIDE) for h in range(2)]
    hist = np.bincount(e[sample], minlength=256)
    order = sorted((b for b in range(256) if hist[b] > 0), key=lambda b: (-int(hist[b]), b))
    syms = order[:RANKS]
    rank = {s: r for r, s in enumerate(syms)}
    # the code shape that is shorter for the sample (mode 1 on a tie)
    cost = {m: sum(int(hist[b]) * _code_of(rank.get(b, RANKS), b, m)[1] for b in order) for m in (1, 2)}
    mode = 2 if cost[2] < cost[1] else 1
    sizes, payload = [], bytearray()
    for t in range(C):
        acc, nb = 0, 0
        for k in range(CHUNK_VALS // 2):
            w = k * C + t
            for h in range(2):
                ex = int(e[2 * w + h])
                code, ln = _code_of(rank.get(ex, RANKS), ex, mode)
                acc |= code << nb
                nb += ln
        nbytes = (nb + 7) // 8
        sizes.append(nbytes)
        payload += acc.to_bytes(nbytes, "little")
    total = (HEADER_BYTES + C + n + len(payload) + 15) // 16 * 16
    raw_total = 16 + 2 * n
    if total >= raw_total:
        hdr = bytearray(16)
        hdr[4:8] = raw_total.to_bytes(4, "little")
        hdr[8:12] = n.to_bytes(4, "little")
        return torch.frombuffer(bytearray(bytes(hdr) + v.astype(np.uint16).tobytes()), dtype=torch.uint8).clone()
    out = bytearray(total)
    out[0], out[1] = mode, len(syms)
    out[2:4] = C.to_bytes(2, "little")
    out[4:8] = total.to_bytes(4, "little")
    out[8:12] = n.to_bytes(4, "little")
    out[16:16 + len(syms)] = bytes(syms)
    out[32:32 + C] = bytes(sizes)
    smb = (((v >> 8) & 0x80) | (v & 0x7F)).astype(np.uint8)
    out[32 + C:32 + C + n] = smb.tobytes()
    out[32 + C + n:32 + C + n + len(payload)] = payload
    return torch.frombuffer(out, dtype=torch.uint8).clone()


def reference_decompress_tile(packed: torch.Tensor) -> torch.Tensor:
    """bf16 values (1-D) of one packed tile, decoded on the CPU from the format description alone."""
    import numpy as np
    b = bytes(packed.reshape(-1).numpy().tobytes())
    mode, total, n = b[0], int.from_bytes(b[4:8], "little"), int.from_bytes(b[8:12], "little")
    assert total == len(b)
    if mode == 0:
        return torch.frombuffer(bytearray(b[16:16 + 2 * n]), dtype=torch.bfloat16).clone()
    C = int.from_bytes(b[2:4], "little")
    syms, sizes = b[16:32], b[32:32 + C]
    smb = np.frombuffer(b[32 + C:32 + C + n], dtype=np.uint8).astype(np.int64)
    e = np.zeros(n, dtype=np.int64)
    off = 32 + C + n
    for t in range(C):
        acc = int.from_bytes(b[off:off + sizes[t]], "little")
        off += sizes[t]
        for k in range(CHUNK_VALS // 2):
            w = k * C + t
            for h in range(2):
                c = acc & 3
                if mode == 2:
                    q = 0
                    while (acc >> q) & 1 and q < FLAT_ESCAPE_ONES:
                        q += 1
                    if q >= FLAT_ESCAPE_ONES:
                        ex, ln = (acc >> FLAT_ESCAPE_ONES) & 0xFF, FLAT_ESCAPE_ONES + 8
                    else:
                        ex, ln = syms[(q << 2) | ((acc >> (q + 1)) & 3)], q + 3
                elif c != 3:
                    ex, ln = syms[c], 2
                else:
                    tt, ones = acc >> 2, 0
                    while (tt >> ones) & 1 and ones < ESCAPE_ONES:
                        ones += 1
                    if ones >= ESCAPE_ONES:
                        ex, ln = (tt >> ESCAPE_ONES) & 0xFF, 2 + ESCAPE_ONES + 8
                    else:
                        ex, ln = syms[SHORT_RANKS + ones], ones + 3
                e[2 * w + h] = ex
                acc >>= ln
    v = ((smb & 0x80) << 8) | (e << 7) | (smb & 0x7F)
    return torch.from_numpy(v.astype(np.uint16).view(np.int16).copy()).view(torch.bfloat16)
