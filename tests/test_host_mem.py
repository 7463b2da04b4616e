"""Host pool allocation: anonymous, huge-page request with fallback, file-backed pools shared
between two mappings (reference: flexkv/storage/allocator.py:190-590, tests/test_config_hugepage.py)."""
import numpy as np

from flexkv_b200 import _native

C = _native.C


def test_anonymous_region_is_zeroed_writable_and_freed():
    r = C.host_region_alloc(3 << 20, populate=True, touch_threads=2)
    a = np.frombuffer(r, dtype=np.uint8)
    assert a.size == 3 << 20 and int(a.sum()) == 0 and not r.file_backed and not r.registered
    a[::4096] = 7
    assert int(a.sum()) == 7 * ((3 << 20) // 4096)
    del a
    r.free()


def test_hugepage_request_falls_back_to_normal_pages_when_none_are_reserved():
    r = C.host_region_alloc(5 << 20, hugepage=True, hugepage_bytes=2 << 20, populate=True, touch_threads=1)
    a = np.frombuffer(r, dtype=np.uint8)
    a[-1] = 9                                   # the whole length is usable either way
    assert r.bytes == 5 << 20 and r.map_bytes >= r.bytes
    assert r.hugepage in (True, False)          # true only where the box has reserved huge pages
    del a
    r.free()


def test_file_backed_pool_is_shared_between_mappings(tmp_path):
    path = str(tmp_path / "pool.bin")
    owner = C.host_region_alloc(1 << 20, populate=True, touch_threads=1, backing_file=path)
    assert owner.file_backed
    a = np.frombuffer(owner, dtype=np.uint8)
    a[:16] = np.arange(16, dtype=np.uint8)
    peer = C.host_region_open(path, 1 << 20)
    b = np.frombuffer(peer, dtype=np.uint8)
    assert b[:16].tolist() == list(range(16))
    b[100] = 42
    assert a[100] == 42
    del a, b
    peer.free()
    owner.free()
