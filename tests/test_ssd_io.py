"""SSD engine: geometry, round trips through io_uring and the thread fallback,
O_DIRECT gating and host-side fault injection (EIO, short IO)."""
import os

import numpy as np
import pytest

from flexkv_b200 import _native

C = _native.C
BLOCK = 8192


def layout(block_first=True, layers=2, kv=2):
    chunk = BLOCK // (layers * kv)
    return dict(cpu_layer_stride=kv * chunk, cpu_kv_stride=chunk, cpu_block_stride=BLOCK, ssd_layer_stride=kv * chunk,
                ssd_kv_stride=chunk, ssd_block_stride=BLOCK, chunk_bytes=chunk, num_layers=layers, kv_dim=kv,
                block_first=block_first)


def engine(tmp_path, ndev=2, files=2, per_file=4, uring=64, direct=True):
    paths = [[str(tmp_path / f"d{d}_f{j}.bin") for j in range(files)] for d in range(ndev)]
    return C.SsdIoEngine(paths, BLOCK, per_file, create=True, try_direct=direct, iouring_entries=uring, num_threads=3), paths


@pytest.mark.parametrize("uring", [64, 0])
@pytest.mark.parametrize("block_first", [True, False])
def test_roundtrip_and_geometry(tmp_path, uring, block_first):
    e, paths = engine(tmp_path, uring=uring)
    assert e.capacity_blocks == 16 and e.using_iouring == (uring > 0)
    for d in paths:
        for f in d:
            assert os.path.getsize(f) == 4 * BLOCK
    region = C.host_region_alloc(16 * BLOCK)
    buf = np.frombuffer(region, dtype=np.uint8)
    rng = np.random.default_rng(0)
    buf[:] = rng.integers(0, 256, size=buf.size, dtype=np.uint8)
    want = buf.copy()
    cpu = np.array([3, 0, 7, 12, 5], dtype=np.int64)
    ssd = np.array([9, 2, 15, 0, 6], dtype=np.int64)
    nfail, ok = e.transfer(region.ptr, cpu, ssd, False, layout(block_first), 0, 2)
    assert nfail == 0 and ok.all()
    # global id -> device = id % ndev, in_dev = id // ndev, file = in_dev % files, slot = in_dev // files
    e.sync_files()
    for c, s in zip(cpu, ssd):
        dev, in_dev = s % 2, s // 2
        f, slot = in_dev % 2, in_dev // 2
        with open(paths[dev][f], "rb") as fh:
            fh.seek(slot * BLOCK)
            assert fh.read(BLOCK) == want[c * BLOCK:(c + 1) * BLOCK].tobytes()
    buf[:] = 0
    cpu2 = np.array([1, 2, 4, 6, 8], dtype=np.int64)
    nfail, ok = e.transfer(region.ptr, cpu2, ssd, True, layout(block_first), 0, 2)
    assert nfail == 0
    for c, c2 in zip(cpu, cpu2):
        assert np.array_equal(buf[c2 * BLOCK:(c2 + 1) * BLOCK], want[c * BLOCK:(c + 1) * BLOCK])
    assert e.bytes_written == 5 * BLOCK and e.bytes_read == 5 * BLOCK
    region.free()


def test_layer_range_moves_only_those_layers(tmp_path):
    e, _ = engine(tmp_path)
    region = C.host_region_alloc(4 * BLOCK)
    buf = np.frombuffer(region, dtype=np.uint8)
    buf[:] = 7
    ids = np.array([0], dtype=np.int64)
    assert e.transfer(region.ptr, ids, ids, False, layout(), 0, 2)[0] == 0
    buf[:] = 0
    assert e.transfer(region.ptr, ids, ids, True, layout(), 1, 1)[0] == 0   # second layer only
    assert buf[:BLOCK // 2].sum() == 0 and (buf[BLOCK // 2:BLOCK] == 7).all()
    region.free()


@pytest.mark.parametrize("uring", [64, 0])
def test_fault_injection(tmp_path, uring):
    e, _ = engine(tmp_path, uring=uring)
    region = C.host_region_alloc(8 * BLOCK)
    buf = np.frombuffer(region, dtype=np.uint8)
    buf[:] = np.random.default_rng(1).integers(0, 256, size=buf.size, dtype=np.uint8)
    want = buf.copy()
    ids = np.arange(4, dtype=np.int64)
    assert e.transfer(region.ptr, ids, ids, False, layout(), 0, 2)[0] == 0
    buf[:] = 0
    e.set_fault(1, 2)                                   # the third IO returns EIO
    nfail, ok = e.transfer(region.ptr, ids, ids, True, layout(), 0, 2)
    assert nfail == 1 and ok.sum() == 3
    for i in np.flatnonzero(ok):
        assert np.array_equal(buf[i * BLOCK:(i + 1) * BLOCK], want[i * BLOCK:(i + 1) * BLOCK])
    buf[:] = 0
    e.set_fault(2, 1)                                   # one IO comes back short and is continued
    nfail, ok = e.transfer(region.ptr, ids, ids, True, layout(), 0, 2)
    assert nfail == 0 and np.array_equal(buf[:4 * BLOCK], want[:4 * BLOCK])
    e.set_fault(3, 0)                                   # everything fails
    nfail, ok = e.transfer(region.ptr, ids, ids, True, layout(), 0, 2)
    assert nfail == 4 and not ok.any()
    e.set_fault(0, 0)
    # ids outside the files are reported, not followed
    nfail, ok = e.transfer(region.ptr, np.array([0, 1], dtype=np.int64), np.array([1, 999], dtype=np.int64), True,
                           layout(), 0, 2)
    assert nfail == 1 and list(ok) == [1, 0]
    region.free()


def test_host_region_file_backed_is_shared(tmp_path):
    f = str(tmp_path / "pool.bin")
    a = C.host_region_alloc(1 << 16, backing_file=f)
    b = C.host_region_open(f, 1 << 16)
    np.frombuffer(a, dtype=np.uint8)[:4] = [1, 2, 3, 4]
    assert list(np.frombuffer(b, dtype=np.uint8)[:4]) == [1, 2, 3, 4]
    assert a.file_backed and not a.registered
    a.free(); b.free()


def test_packed_blocks_move_only_their_used_bytes(tmp_path):
    """Host blocks in the lossless codec's slot format: tile slots of which only the first size bytes are used.
    A packed write gathers them into one run per block, the read scatters them back; the bytes on the SSD
    interface are the used bytes rounded up to 4 KiB, and a corrupt size row fails only its block."""
    tile_slot, last_slot, tpc, chunks = 4096 + 128, 2048 + 128, 2, 3          # chunk = one full and one short tile
    chunk_slot = tile_slot + last_slot
    block = 32768                                                               # 4 KiB multiple >= chunks * chunk_slot
    assert chunks * chunk_slot <= block
    paths = [[str(tmp_path / "p0.bin"), str(tmp_path / "p1.bin")]]
    e = C.SsdIoEngine(paths, block, 4, create=True, try_direct=True, iouring_entries=32, num_threads=2)
    region = C.host_region_alloc(8 * block)
    buf = np.frombuffer(region, dtype=np.uint8)
    rng = np.random.default_rng(3)
    buf[:] = rng.integers(0, 256, size=buf.size, dtype=np.uint8)
    geo = dict(cpu_block_stride=block, chunk_slot_bytes=chunk_slot, tile_slot_bytes=tile_slot,
               last_tile_slot_bytes=last_slot, tiles_per_chunk=tpc, entries=chunks * tpc)
    cpu = np.array([1, 5, 6], dtype=np.int64)
    ssd = np.array([7, 0, 3], dtype=np.int64)
    sizes = rng.integers(2, 64, size=(3, chunks * tpc)).astype(np.int32) * 16      # multiples of 16 under every slot
    want = buf.copy()
    nfail, ok = e.transfer_packed(region.ptr, cpu, ssd, False, geo, sizes)
    assert nfail == 0 and ok.all()
    written = int(sum((int(r.sum()) + 4095) // 4096 * 4096 for r in sizes))
    assert e.bytes_written == written < 3 * block
    buf[:] = 0
    cpu2 = np.array([0, 2, 4], dtype=np.int64)
    nfail, ok = e.transfer_packed(region.ptr, cpu2, ssd, True, geo, sizes)
    assert nfail == 0 and e.bytes_read == written
    for i in range(3):
        for t in range(chunks * tpc):
            off = (t // tpc) * chunk_slot + (t % tpc) * tile_slot
            a = buf[cpu2[i] * block + off:cpu2[i] * block + off + sizes[i, t]]
            b = want[cpu[i] * block + off:cpu[i] * block + off + sizes[i, t]]
            assert np.array_equal(a, b), (i, t)
    # a row with an impossible size fails its block and nothing else
    bad = sizes.copy()
    bad[1, 3] = last_slot + 16
    nfail, ok = e.transfer_packed(region.ptr, cpu, ssd, False, geo, bad)
    assert nfail == 1 and list(ok) == [1, 0, 1]
    e.set_fault(3, 0)
    nfail, ok = e.transfer_packed(region.ptr, cpu2, ssd, True, geo, sizes)
    assert nfail == 3
    e.set_fault(0, 0)
    region.free()
