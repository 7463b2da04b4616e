"""Codec strategies used by the GPU<->host workers.

A strategy is attached once to a worker (``attach``) and then launches one fused
pack-or-unpack kernel per rank and op (``run``). Reference plug-in point:
flexkv/transfer/compression/common/strategy.py:13-51 (``CompressionStrategy.attach/run``,
``NullCompressionStrategy``); the nvCOMP ANS strategy of the reference
(compression/ans/ans_strategy.py) is replaced by own kernels: no staging buffer and no
second pass, the copy kernel itself reads GPU pages and writes packed host tiles.
"""
from __future__ import annotations

from typing import Any, Dict

from ... import _native


class CompressionStrategy:
    """Interface. ``params`` is the addressing dict of one rank's launch (same keys as
    the plain copy kernel); ``stream`` is a raw CUDA stream handle."""
    name = "abstract"
    lossless = True

    def attach(self, worker: Any) -> None:
        self.worker = worker

    def host_chunk_bytes(self, chunk_elems: int, itemsize: int) -> int:
        raise NotImplementedError

    def run(self, params: Dict[str, Any], rank_index: int, num_ctas: int, stream: int) -> None:
        raise NotImplementedError

    @property
    def needs_size_table(self) -> bool:
        return False


class NullCompressionStrategy(CompressionStrategy):
    """Raw bytes through the plain copy kernel (used when every codec is refused)."""
    name = "none"

    def host_chunk_bytes(self, chunk_elems: int, itemsize: int) -> int:
        return chunk_elems * itemsize

    def run(self, params, rank_index, num_ctas, stream) -> None:
        _native.C.kv_copy(params, num_ctas, int(params.get("tile_bytes", 16384)), 0, stream)


class Fp8BlockScaleStrategy(CompressionStrategy):
    """bf16/fp16 -> fp8 e4m3 with one fp32 scale per 128 values (lossy, 0.53x bytes)."""
    name = "fp8_e4m3"
    lossless = False
    GROUP = 128

    def host_chunk_bytes(self, chunk_elems: int, itemsize: int) -> int:
        if chunk_elems % self.GROUP:
            raise ValueError("fp8 offload needs chunk elements divisible by 128")
        return chunk_elems + (chunk_elems // self.GROUP) * 4

    def run(self, params, rank_index, num_ctas, stream) -> None:
        _native.C.kv_quant_fp8(params, num_ctas, stream)


class ExponentPackStrategy(CompressionStrategy):
    """Lossless bf16 codec: sign+mantissa bytes stay raw, every group of 128 values stores its
    largest exponent once and each value's distance to it in w bits, w chosen per group
    (about 0.75x bytes on unit-normal data)."""
    name = "bf16_xp"
    TILE_ELEMS = 8192
    TILE_SLOT = 2 * TILE_ELEMS + 128

    def __init__(self, size_table=None, spec=None) -> None:
        self.size_table = size_table
        self.spec = spec

    @property
    def needs_size_table(self) -> bool:
        return True

    def host_chunk_bytes(self, chunk_elems: int, itemsize: int) -> int:
        if chunk_elems % 1024:
            raise ValueError("the exponent-packing codec needs chunk elements divisible by 1024")
        full, rest = divmod(chunk_elems, self.TILE_ELEMS)
        return full * self.TILE_SLOT + ((2 * rest + 128) if rest else 0)

    def run(self, params, rank_index, num_ctas, stream) -> None:
        if self.size_table is None or self.spec is None:
            raise RuntimeError("exponent-packing strategy used without a size table")
        off = self.spec.rank_offset_entries(rank_index)
        _native.C.kv_compress_bf16(params, self.size_table.data_ptr() + 4 * off, self.spec.kernel_layers(), num_ctas,
                                   stream)


def strategy_for(codec: str, size_table=None, spec=None) -> CompressionStrategy:
    if codec == "fp8_e4m3":
        return Fp8BlockScaleStrategy()
    if codec == "bf16_xp":
        return ExponentPackStrategy(size_table, spec)
    if codec == "none":
        return NullCompressionStrategy()
    raise ValueError(f"unknown host codec {codec!r}")
