"""Per-tile size tables of the lossless codec.

The host slot geometry never changes: every (block, layer, kv) chunk keeps a full-size
slot and a compressed tile occupies the first ``size`` bytes of its tile slot. ``size``
lives in an int32 table with one entry per tile, canonical shape
``[blocks, layers, kv, tiles]`` when one rank writes a chunk (tp == 1 or shared KV) and
``[blocks, tp, layers, kv, tiles]`` otherwise — the rank axis sits right after the
block axis so that one block's entries stay contiguous and move to the SSD table with a
single row copy (reference: flexkv/transfer/compression/common/size_table.py:10-32 and
flexkv/transfer/compression/ans/ans_utils.py:159-239; ``H2DISK: ssd[s] = cpu[c]``,
``DISK2H: cpu[c'] = ssd[s]``, tables are not persisted, ans_utils.py:215-219).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import numpy as np


@dataclass(frozen=True)
class SizeTableSpec:
    num_blocks: int
    num_layers: int
    kv_dim: int
    tiles_per_chunk: int
    tp: int = 1                      # 1 = canonical

    @property
    def shape(self) -> Tuple[int, ...]:
        if self.tp == 1:
            return (self.num_blocks, self.num_layers, self.kv_dim, self.tiles_per_chunk)
        return (self.num_blocks, self.tp, self.num_layers, self.kv_dim, self.tiles_per_chunk)

    @property
    def entries_per_block(self) -> int:
        return self.tp * self.num_layers * self.kv_dim * self.tiles_per_chunk

    def rank_offset_entries(self, rank: int) -> int:
        """Offset of rank ``rank``'s first entry inside one block's row."""
        return 0 if self.tp == 1 else rank * self.num_layers * self.kv_dim * self.tiles_per_chunk

    def kernel_layers(self) -> int:
        """What the kernel is told the table's layer extent is: a rank walks a table of
        tp * layers "layers" starting ``rank_offset_entries`` in."""
        return self.tp * self.num_layers

    def alloc(self, pinned: bool = False):
        import torch
        t = torch.zeros(self.shape, dtype=torch.int32)
        return t.pin_memory() if pinned else t

    def alloc_ssd(self, num_ssd_blocks: int) -> np.ndarray:
        return np.zeros((num_ssd_blocks, self.entries_per_block), dtype=np.int32)


def copy_rows(dst: np.ndarray, dst_blocks: np.ndarray, src: np.ndarray, src_blocks: np.ndarray) -> None:
    """``dst[dst_blocks] = src[src_blocks]`` on tables flattened to [blocks, entries]."""
    d = dst.reshape(dst.shape[0], -1)
    s = src.reshape(src.shape[0], -1)
    d[np.asarray(dst_blocks, dtype=np.int64)] = s[np.asarray(src_blocks, dtype=np.int64)]
