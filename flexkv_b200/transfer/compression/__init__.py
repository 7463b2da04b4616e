"""Host-tier codecs as pluggable strategies (reference: flexkv/transfer/compression/*).

* ``strategy``   ``CompressionStrategy`` interface plus the null, block-scaled fp8 and
                 lossless exponent-packing strategies (each one wraps an sm_100a kernel
                 that packs on the way out of the GPU and unpacks on the way in);
* ``policy``     the enable rules (all-or-nothing across tiers);
* ``size_table`` shapes and indexing of the per-tile size tables;
* ``factory``    ``build_compressors`` used by the GPU<->host workers.
"""
from .factory import build_compressors
from .policy import CodecDecision, choose_codec
from .size_table import SizeTableSpec
from .strategy import (CompressionStrategy, ExponentPackStrategy, Fp8BlockScaleStrategy, NullCompressionStrategy)

__all__ = ["build_compressors", "CodecDecision", "choose_codec", "SizeTableSpec", "CompressionStrategy",
           "ExponentPackStrategy", "Fp8BlockScaleStrategy", "NullCompressionStrategy"]
