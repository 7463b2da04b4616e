"""When a host-tier codec may be switched on.

All-or-nothing: if the codec is refused, GPU<->host and host<->SSD both run raw
(reference rules: flexkv/transfer/compression/ans/ans_utils.py:19-29,51-118,276-282).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ...common.storage import KVCacheLayoutType

MIN_CHUNK_BYTES = 4096          # below this the fixed per-tile cost dominates
SMALL_CHUNK_WARN_BYTES = 16384  # ratio plateaus from here up
XP_ELEM_MULTIPLE = 1024         # lossless codec: chunk elements per rank
FP8_ELEM_MULTIPLE = 512         # block-scaled fp8: chunk elements per rank


@dataclass(frozen=True)
class CodecDecision:
    codec: str                      # none | fp8_e4m3 | bf16_xp
    reason: str = ""                # why compression was refused (codec == "none" although requested)
    warning: str = ""


def choose_codec(*, requested_quant: str, compression_enabled: bool, dtype, host_layout_type, chunk_elems_per_rank: int,
                 itemsize: int, layerwise: bool, peer_host_sharing: bool = False,
                 pipeline_stages: int = 1) -> CodecDecision:
    """``requested_quant`` is the explicit lossy choice (CacheConfig.offload_quant); the
    lossless codec is picked when compression is enabled and the cache qualifies."""
    if requested_quant not in ("none", "fp8_e4m3", "bf16_xp"):
        raise ValueError(f"unknown host codec {requested_quant!r}")
    chunk_bytes = chunk_elems_per_rank * itemsize
    if pipeline_stages > 1 and (requested_quant != "none" or compression_enabled):
        return CodecDecision("none", "several pipeline stages share one host block (codecs address whole blocks)")
    if requested_quant == "fp8_e4m3":
        if dtype not in (torch.bfloat16, torch.float16):
            return CodecDecision("none", f"fp8 offload needs a 16-bit cache, got {dtype}")
        if chunk_elems_per_rank % FP8_ELEM_MULTIPLE:
            return CodecDecision("none", f"chunk elements per rank not a multiple of {FP8_ELEM_MULTIPLE}")
        if host_layout_type != KVCacheLayoutType.BLOCKFIRST:
            return CodecDecision("none", "host layout is not BLOCKFIRST")
        if layerwise:
            return CodecDecision("none", "layerwise restore consumes raw host blocks")
        return CodecDecision("fp8_e4m3")
    if requested_quant == "none" and not compression_enabled:
        return CodecDecision("none")
    why: Optional[str] = None
    if dtype != torch.bfloat16:
        why = f"dtype {dtype} is not bf16"
    elif host_layout_type != KVCacheLayoutType.BLOCKFIRST:
        why = "host layout is not BLOCKFIRST"
    elif chunk_bytes < MIN_CHUNK_BYTES:
        why = f"chunks of {chunk_bytes} B are below {MIN_CHUNK_BYTES} B"
    elif chunk_elems_per_rank % XP_ELEM_MULTIPLE:
        why = f"chunk elements per rank are not a multiple of {XP_ELEM_MULTIPLE}"
    elif peer_host_sharing:
        why = "host blocks are shared with other nodes (the size table is not)"
    if why:
        return CodecDecision("none", why)
    warn = ""
    if chunk_bytes < SMALL_CHUNK_WARN_BYTES:
        warn = f"chunks of {chunk_bytes} B are small for the lossless codec; expect a weaker ratio"
    return CodecDecision("bf16_xp", warning=warn)
