"""KV block layouts: shapes and byte strides of a pool on any tier.

Three orderings of the same six axes ``(L layers, K kv planes, B blocks,
T tokens per block, H heads, D head size)`` are supported, with the same
meaning as the reference's ``KVCacheLayoutType``
(flexkv/common/storage.py:26-150,203-247):

* ``LAYERFIRST``  ``[L, K, B, T, H, D]``
* ``BLOCKFIRST``  ``[B, L, K, T, H, D]``  (host / SSD block format)
* ``LAYERBLOCK``  ``[L, B, K, T, H, D]``

A *chunk* is the contiguous ``T*H*D`` run that every layout keeps intact; the
copy kernels move chunks and never look inside them. Heterogeneous layer
groups are stored byte-flat, block first, groups concatenated in order
(flexkv/common/storage.py:87-127,249-286).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Tuple

import torch


class KVCacheLayoutType(Enum):
    LAYERFIRST = "LAYERFIRST"
    BLOCKFIRST = "BLOCKFIRST"
    LAYERBLOCK = "LAYERBLOCK"


class AccessHandleType(Enum):
    TENSOR = "tensor"            # torch tensor(s) in this process
    TENSOR_HANDLE = "handle"     # exported handle(s) of another process' tensors
    FILE = "file"                # list of files
    HOST_REGION = "host_region"  # native host pool


@dataclass
class GroupLayout:
    """One homogeneous layer group inside a byte-flat multi-group block."""
    num_layers: int
    kv_dim: int
    tokens_per_block: int       # already divided by the group's compress ratio
    num_heads: int
    head_size: int
    itemsize: int
    offset_bytes: int = 0       # start of the group inside one rank's slice of the block

    @property
    def chunk_bytes(self) -> int:
        return self.tokens_per_block * self.num_heads * self.head_size * self.itemsize

    @property
    def layer_stride_bytes(self) -> int:
        return self.kv_dim * self.chunk_bytes

    @property
    def bytes(self) -> int:
        return self.num_layers * self.layer_stride_bytes


@dataclass(init=False)
class KVCacheLayout:
    type: KVCacheLayoutType
    num_layer: int
    num_block: int
    tokens_per_block: int
    num_head: int
    head_size: int
    is_mla: bool = False
    kv_dim_override: Optional[int] = None
    groups: Optional[List[GroupLayout]] = None   # byte-flat multi-group block (BLOCKFIRST only)
    tp_slices: int = 1                           # multi-group: rank slices per block

    def __init__(self, type: KVCacheLayoutType, num_layer: int, num_block: int, tokens_per_block: int, num_head: int,
                 head_size: int, is_mla=False, kv_dim_override: Optional[int] = None,
                 groups: Optional[List[GroupLayout]] = None, tp_slices: int = 1, *, kv_dim: Optional[int] = None,
                 num_kv_heads: Optional[int] = None) -> None:
        """Also takes the reference's spelling (flexkv/common/storage.py:31-48): ``kv_dim`` (1 for an MLA latent
        cache or a packed 4-D cache, 2 for K and V) as a keyword or as the seventh positional argument, and
        ``num_kv_heads``, which is kept for the caller and not used here."""
        if not isinstance(is_mla, bool) and isinstance(is_mla, int):       # positional kv_dim of the reference
            kv_dim, is_mla = int(is_mla), False
        if kv_dim is not None:
            kv_dim_override = int(kv_dim)
            is_mla = bool(is_mla) or (kv_dim_override == 1 and int(num_head) == 1)
        if kv_dim_override is not None and kv_dim_override == (1 if is_mla else 2):
            kv_dim_override = None                   # the implied value: keeps equal layouts equal
        self.type, self.num_layer, self.num_block = type, int(num_layer), int(num_block)
        self.tokens_per_block, self.num_head, self.head_size = int(tokens_per_block), int(num_head), int(head_size)
        self.is_mla, self.kv_dim_override, self.groups, self.tp_slices = bool(is_mla), kv_dim_override, groups, tp_slices
        self.num_kv_heads = num_kv_heads
        self.__post_init__()

    def __post_init__(self) -> None:
        if self.groups is not None and self.type != KVCacheLayoutType.BLOCKFIRST:
            raise ValueError("multi-group layouts are byte-flat BLOCKFIRST only")
        if self.groups is not None:
            off = 0
            for g in self.groups:
                g.offset_bytes = off
                off += g.bytes

    # ---- element-space geometry -------------------------------------------------
    @property
    def kv_dim(self) -> int:
        if self.kv_dim_override is not None:
            return self.kv_dim_override
        return 1 if self.is_mla else 2

    @property
    def is_multi_group(self) -> bool:
        return self.groups is not None

    @property
    def kv_shape(self) -> torch.Size:
        L, K, B, T, H, D = (self.num_layer, self.kv_dim, self.num_block, self.tokens_per_block,
                            self.num_head, self.head_size)
        if self.groups is not None:
            return torch.Size([B, self.block_bytes_flat])
        if self.type == KVCacheLayoutType.LAYERFIRST:
            return torch.Size([L, K, B, T, H, D])
        if self.type == KVCacheLayoutType.BLOCKFIRST:
            return torch.Size([B, L, K, T, H, D])
        return torch.Size([L, B, K, T, H, D])

    @property
    def block_bytes_flat(self) -> int:
        assert self.groups is not None
        return self.tp_slices * sum(g.bytes for g in self.groups)

    def get_chunk_size(self) -> int:
        return self.tokens_per_block * self.num_head * self.head_size

    def get_total_elements(self) -> int:
        if self.groups is not None:
            return self.num_block * self.block_bytes_flat
        return self.num_layer * self.kv_dim * self.num_block * self.get_chunk_size()

    def get_elements_per_block(self) -> int:
        if self.groups is not None:
            return self.block_bytes_flat
        return self.num_layer * self.kv_dim * self.get_chunk_size()

    def get_layer_stride(self) -> int:
        c = self.get_chunk_size()
        if self.type == KVCacheLayoutType.LAYERFIRST:
            return self.kv_dim * self.num_block * c
        if self.type == KVCacheLayoutType.BLOCKFIRST:
            return self.kv_dim * c
        return self.num_block * self.kv_dim * c

    def get_block_stride(self) -> int:
        c = self.get_chunk_size()
        if self.groups is not None:
            return self.block_bytes_flat
        if self.type == KVCacheLayoutType.LAYERFIRST:
            return c
        if self.type == KVCacheLayoutType.BLOCKFIRST:
            return self.num_layer * self.kv_dim * c
        return self.kv_dim * c

    def get_kv_stride(self) -> int:
        c = self.get_chunk_size()
        if self.type == KVCacheLayoutType.LAYERFIRST:
            return self.num_block * c
        return c

    # ---- derived layouts --------------------------------------------------------
    def div_block(self, n: int, padding: bool = False) -> "KVCacheLayout":
        nb = (self.num_block + n - 1) // n if padding else self.num_block // n
        return self._replace(num_block=nb)

    def div_layer(self, n: int) -> "KVCacheLayout":
        if self.num_layer % n:
            raise ValueError("layers not divisible")
        return self._replace(num_layer=self.num_layer // n)

    def div_head(self, n: int) -> "KVCacheLayout":
        """Per-rank view of a pool that concatenates the heads of ``n`` ranks."""
        if self.is_mla or self.num_head == 1:
            return self._replace()
        if self.num_head % n:
            raise ValueError("heads not divisible")
        return self._replace(num_head=self.num_head // n)

    def _replace(self, **kw) -> "KVCacheLayout":
        d = dict(type=self.type, num_layer=self.num_layer, num_block=self.num_block,
                 tokens_per_block=self.tokens_per_block, num_head=self.num_head, head_size=self.head_size,
                 is_mla=self.is_mla, kv_dim_override=self.kv_dim_override, groups=self.groups,
                 tp_slices=self.tp_slices)
        d.update(kw)
        return KVCacheLayout(**d)

    def byte_strides(self, itemsize: int) -> Tuple[int, int, int, int]:
        """``(layer, kv, block, chunk)`` strides in bytes."""
        if self.groups is not None:
            raise ValueError("multi-group layouts have per-group strides; use group_byte_strides")
        return (self.get_layer_stride() * itemsize, self.get_kv_stride() * itemsize,
                self.get_block_stride() * itemsize, self.get_chunk_size() * itemsize)

    def group_byte_strides(self, g: int) -> Tuple[int, int, int, int, int]:
        """``(offset, layer, kv, block, chunk)`` byte strides of group ``g``."""
        assert self.groups is not None
        grp = self.groups[g]
        return (grp.offset_bytes, grp.layer_stride_bytes, grp.chunk_bytes, self.block_bytes_flat, grp.chunk_bytes)


@dataclass
class StorageHandle:
    handle_type: AccessHandleType
    data: object
    kv_layout: KVCacheLayout
    dtype: torch.dtype
    gpu_device_id: Optional[int] = None
    num_blocks_per_file: Optional[int] = None
    remote_config_custom: Optional[dict] = None

    def get_tensor(self):
        assert self.handle_type == AccessHandleType.TENSOR
        return self.data

    def get_file_list(self) -> List[str]:
        assert self.handle_type == AccessHandleType.FILE
        return self.data  # type: ignore[return-value]
