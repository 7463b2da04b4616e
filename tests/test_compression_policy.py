"""Enable rules, size-table shapes and strategy selection of the host codecs
(reference rules: flexkv/transfer/compression/ans/ans_utils.py:19-118,159-239)."""
import numpy as np
import torch

from flexkv_b200.common.storage import KVCacheLayoutType
from flexkv_b200.transfer.compression import (ExponentPackStrategy, Fp8BlockScaleStrategy, NullCompressionStrategy,
                                              SizeTableSpec, choose_codec)
from flexkv_b200.transfer.compression.size_table import copy_rows
from flexkv_b200.transfer.compression.strategy import strategy_for

BF = KVCacheLayoutType.BLOCKFIRST


def _dec(**kw):
    base = dict(requested_quant="none", compression_enabled=True, dtype=torch.bfloat16, host_layout_type=BF,
                chunk_elems_per_rank=16384, itemsize=2, layerwise=False)
    base.update(kw)
    return choose_codec(**base)


def test_lossless_codec_is_all_or_nothing():
    assert _dec().codec == "bf16_xp"
    assert _dec(compression_enabled=False).codec == "none" and not _dec(compression_enabled=False).reason
    for kw, word in [(dict(dtype=torch.float16), "bf16"), (dict(host_layout_type=KVCacheLayoutType.LAYERFIRST), "BLOCKFIRST"),
                     (dict(chunk_elems_per_rank=1024), "below"), (dict(chunk_elems_per_rank=16384 + 512), "multiple")]:
        d = _dec(**kw)
        assert d.codec == "none" and word in d.reason, (kw, d)
    assert "small" in _dec(chunk_elems_per_rank=4096).warning
    # the layer-by-layer restore has a form of the unpacking kernel; the lossy fp8 format has not
    assert _dec(layerwise=True).codec == "bf16_xp"
    assert "layerwise" in _dec(requested_quant="fp8_e4m3", compression_enabled=False, layerwise=True).reason


def test_fp8_is_explicit_and_checked():
    assert _dec(requested_quant="fp8_e4m3", compression_enabled=False).codec == "fp8_e4m3"
    assert _dec(requested_quant="fp8_e4m3", dtype=torch.uint8).codec == "none"
    assert _dec(requested_quant="fp8_e4m3", chunk_elems_per_rank=640).codec == "none"


def test_size_table_shapes_and_row_moves():
    canon = SizeTableSpec(10, 4, 2, 3)
    assert canon.shape == (10, 4, 2, 3) and canon.entries_per_block == 24 and canon.rank_offset_entries(0) == 0
    tp = SizeTableSpec(10, 4, 2, 3, tp=2)
    assert tp.shape == (10, 2, 4, 2, 3) and tp.entries_per_block == 48
    assert tp.rank_offset_entries(1) == 24 and tp.kernel_layers() == 8
    cpu = tp.alloc().numpy()
    cpu[:] = np.arange(cpu.size, dtype=np.int32).reshape(cpu.shape)
    ssd = tp.alloc_ssd(6)
    copy_rows(ssd, [5, 0], cpu, [2, 9])              # H2DISK: ssd[s] = cpu[c]
    assert (ssd[5] == cpu[2].reshape(-1)).all() and (ssd[0] == cpu[9].reshape(-1)).all()
    back = np.zeros_like(cpu)
    copy_rows(back, [7], ssd, [5])                   # DISK2H: cpu[c'] = ssd[s]
    assert (back[7] == cpu[2]).all()


def test_strategy_geometry():
    assert isinstance(strategy_for("none"), NullCompressionStrategy)
    f = strategy_for("fp8_e4m3")
    assert isinstance(f, Fp8BlockScaleStrategy) and not f.lossless
    assert f.host_chunk_bytes(16384, 2) == 16384 + 128 * 4
    x = strategy_for("bf16_xp")
    assert isinstance(x, ExponentPackStrategy) and x.lossless and x.needs_size_table
    assert x.host_chunk_bytes(16384, 2) == 2 * (2 * 8192 + 128)
