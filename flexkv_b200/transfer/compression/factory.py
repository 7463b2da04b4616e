"""Builds the codec strategy of a host pool (reference: flexkv/transfer/compression/factory.py:23-68)."""
from __future__ import annotations

from typing import Optional

from .size_table import SizeTableSpec
from .strategy import CompressionStrategy, strategy_for


def build_compressors(host_pool, num_layers: int, kv_dim: int, tp: int, shared_kv: bool) -> CompressionStrategy:
    """``host_pool`` is the storage engine's HostPool: its ``quant`` field names the codec
    decided at allocation time and ``size_table`` holds the lossless codec's sizes."""
    codec = getattr(host_pool, "quant", "none") or "none"
    spec: Optional[SizeTableSpec] = None
    if codec == "bf16_xp":
        spec = SizeTableSpec(host_pool.num_blocks, num_layers, kv_dim, host_pool.tiles_per_chunk,
                             tp=1 if shared_kv else tp)
    return strategy_for(codec, getattr(host_pool, "size_table", None), spec)
