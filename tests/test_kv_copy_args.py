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
