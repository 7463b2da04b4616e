"""Argument checks of the copy paths that run before anything touches memory: the tensor tables must
cover every (layer, kv plane) a call addresses. Exercised on the CPU through the host restatement of the
kernel's addressing, which shares the check with every launch path."""
import numpy as np

from flexkv_b200 import _native

C = _native.C
KV_ERR_BAD_ARGS = 8


def _params(num_ptrs, num_layers=4, kv_dim=2, idx_layer_mul=1, idx_kv_mul=0, holes=()):
    chunk = 64
    gpu = np.zeros((num_layers, kv_dim, 8, chunk), dtype=np.uint8)
    cpu = np.zeros((8, num_layers, kv_dim, chunk), dtype=np.uint8)
    gpu[:] = np.arange(gpu.size, dtype=np.uint64).reshape(gpu.shape) % 251
    ptrs = [gpu[l].ctypes.data for l in range(num_layers)][:num_ptrs]
    for h in holes:
        ptrs[h] = 0
    g = np.array([1, 5], dtype=np.int64)
    c = np.array([7, 0], dtype=np.int64)
    p = dict(gpu_ptrs=ptrs, idx_layer_mul=idx_layer_mul, idx_kv_mul=idx_kv_mul, g_kv_stride=8 * chunk,
             g_block_stride=chunk, cpu_base=cpu.ctypes.data, c_layer_stride=kv_dim * chunk, c_kv_stride=chunk,
             c_block_stride=num_layers * kv_dim * chunk, gpu_blocks_ptr=g.ctypes.data, cpu_blocks_ptr=c.ctypes.data,
             num_pairs=2, layer_start=0, num_layers=num_layers, kv_dim=kv_dim, chunk_bytes=chunk,
             gpu_num_blocks=8, cpu_num_blocks=8, h2d=0)
    return p, gpu, cpu, (g, c)


def test_full_table_copies_and_short_table_is_refused():
    p, gpu, cpu, keep = _params(4)
    assert C.host_kv_copy(p, 1) == 0
    assert np.array_equal(cpu[7, 2, 1], gpu[2, 1, 1]) and np.array_equal(cpu[0, 3, 0], gpu[3, 0, 5])
    p, gpu, cpu, keep = _params(3)                       # 4 layers address entries 0..3, only 3 were given
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    assert not cpu.any()                                 # nothing was written


def test_wrong_multipliers_and_null_entries_are_refused():
    p, gpu, cpu, keep = _params(4, idx_layer_mul=2)      # last index 6 is past the table
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    p, gpu, cpu, keep = _params(4, idx_kv_mul=4)         # SGLang-style plane offset with a vLLM-sized table
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    p, gpu, cpu, keep = _params(4, holes=(2,))           # a tensor that was never re-registered
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    p, gpu, cpu, keep = _params(4, idx_layer_mul=-1)
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    assert not cpu.any()


def _big_params(num_layers, holes=(), short=0):
    """SGLang-style registration: all K tensors, then all V tensors, one per layer."""
    chunk, nb = 32, 4
    gpu = np.zeros((2 * num_layers, nb, chunk), dtype=np.uint8)
    gpu[:] = (np.arange(gpu.size, dtype=np.uint64).reshape(gpu.shape) * 7) % 253
    cpu = np.zeros((nb, num_layers, 2, chunk), dtype=np.uint8)
    ptrs = [gpu[i].ctypes.data for i in range(2 * num_layers)]
    ptrs = ptrs[:len(ptrs) - short]
    for h in holes:
        ptrs[h] = 0
    g = np.array([3, 0, 2], dtype=np.int64)
    c = np.array([1, 2, 0], dtype=np.int64)
    p = dict(gpu_ptrs=ptrs, idx_layer_mul=1, idx_kv_mul=num_layers, g_block_stride=chunk, cpu_base=cpu.ctypes.data,
             c_layer_stride=2 * chunk, c_kv_stride=chunk, c_block_stride=num_layers * 2 * chunk,
             gpu_blocks_ptr=g.ctypes.data, cpu_blocks_ptr=c.ctypes.data, num_pairs=3, layer_start=0,
             num_layers=num_layers, kv_dim=2, chunk_bytes=chunk, gpu_num_blocks=nb, cpu_num_blocks=nb, h2d=0)
    return p, gpu, cpu, (g, c)


def test_more_tensors_than_the_inline_table_holds():
    """320 tensors (160 layers, K and V apart) exceed the 256 pointers that travel inside the launch parameters:
    the table then lives in memory of its own and the same addressing and the same checks apply."""
    L = 160
    assert 2 * L > C.MAX_GPU_PTRS and 2 * L <= C.MAX_GPU_PTRS_EXT
    p, gpu, cpu, keep = _big_params(L)
    before = C.ptr_table_cache_size()
    assert C.kv_copy_tma_eligible(p)
    assert C.host_kv_copy(p, 2) == 0
    for pair, (gb, cb) in enumerate(zip(*keep)):
        for l in (0, 1, 127, 128, 159):
            assert np.array_equal(cpu[cb, l, 0], gpu[l, gb]) and np.array_equal(cpu[cb, l, 1], gpu[L + l, gb])
    assert C.ptr_table_cache_size() == before + 1
    assert C.host_kv_copy(p, 2) == 0                       # the same registration reuses its table
    assert C.ptr_table_cache_size() == before + 1
    # and back: scatter host blocks into a second paged cache through a layer window of the same large table
    gpu2 = np.zeros_like(gpu)
    p2 = dict(p, gpu_ptrs=[gpu2[i].ctypes.data for i in range(2 * L)], h2d=1, layer_start=100, num_layers=60)
    assert C.host_kv_copy(p2, 2) == 0
    g, c = keep
    assert np.array_equal(gpu2[130, g[0]], gpu[130, g[0]]) and np.array_equal(gpu2[L + 159, g[2]], gpu[L + 159, g[2]])
    assert not gpu2[99].any() and not gpu2[L + 99].any()   # layers outside the window stay untouched


def test_large_table_is_checked_like_the_inline_one():
    p, gpu, cpu, keep = _big_params(160, short=1)          # last V tensor missing
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    p, gpu, cpu, keep = _big_params(160, holes=(300,))
    assert C.host_kv_copy(p, 1) == KV_ERR_BAD_ARGS
    assert not cpu.any()
    p, gpu, cpu, keep = _big_params(160)
    p["gpu_ptrs"] = p["gpu_ptrs"] * 60                     # 19 200 entries: past the table limit
    try:
        C.host_kv_copy(p, 1)
        raise AssertionError("accepted an oversized table")
    except ValueError:
        pass
