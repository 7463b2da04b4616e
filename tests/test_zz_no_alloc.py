"""The allocation-free restore entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when a restore is due:
the engine has already given all free HBM to its KV pool, or the calling thread
must not take the device-wide synchronisation that cudaMalloc implies. For them
``fkv_layerwise_copy_noalloc`` keeps the kernel's per-layer completion counters
in a fixed array inside the library. This test drives that symbol with ctypes
and checks, on two calls in a row (the array is shared and keeps its contents
between calls), that the restored bytes and the published flags are exactly
those of the ordinary entry point, whose scratch is a caller-provided tensor.
The file sorts last so that a failure here cannot hide any other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from flexkv_b200 import _native
from flexkv_b200.models import KVShape, alloc_paged_cache
from flexkv_b200.ops.kv_copy import HostSide, decode_status, make_params, new_status
from flexkv_b200.storage.gpu_layout import register_tensors

pytestmark = pytest.mark.gpu


class Args(ctypes.Structure):
    _fields_ = [("gpu_ptrs", ctypes.POINTER(ctypes.c_uint64)), ("num_gpu_ptrs", ctypes.c_int32),
                ("idx_layer_mul", ctypes.c_int32), ("idx_kv_mul", ctypes.c_int32),
                ("g_layer_stride", ctypes.c_int64), ("g_kv_stride", ctypes.c_int64), ("g_block_stride", ctypes.c_int64),
                ("cpu_base", ctypes.c_uint64), ("c_layer_stride", ctypes.c_int64), ("c_kv_stride", ctypes.c_int64),
                ("c_block_stride", ctypes.c_int64), ("c_off", ctypes.c_int64),
                ("gpu_blocks", ctypes.c_void_p), ("cpu_blocks", ctypes.c_void_p), ("num_pairs", ctypes.c_int32),
                ("num_layers", ctypes.c_int32), ("kv_dim", ctypes.c_int32), ("chunk_bytes", ctypes.c_int64),
                ("gpu_num_blocks", ctypes.c_int64), ("cpu_num_blocks", ctypes.c_int64),
                ("dev_flags", ctypes.c_void_p), ("host_flags", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("epoch", ctypes.c_uint32), ("num_ctas", ctypes.c_int32), ("tile_bytes", ctypes.c_int32)]


def _entry():
    lib = ctypes.CDLL(_native.C.__file__)
    fn = lib.fkv_layerwise_copy_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(Args), ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _args(reg, host, g, c, flags, status, epoch, num_layers):
    ptrs = (ctypes.c_uint64 * len(reg.ptrs))(*[int(p) for p in reg.ptrs])
    a = Args(ptrs, len(reg.ptrs), reg.idx_layer_mul, reg.idx_kv_mul, reg.layer_stride, reg.kv_stride,
             reg.block_stride, host.base, host.layer_stride, host.kv_stride, host.block_stride, 0,
             g.data_ptr(), c.data_ptr(), g.numel(), num_layers, reg.kv_dim, reg.chunk_bytes, reg.num_blocks,
             host.num_blocks, flags.data_ptr(), None, status.data_ptr(), epoch, 6, 4096)
    a._keep = ptrs
    return a


def test_noalloc_entry_matches_the_ordinary_one_twice_in_a_row():
    dev = torch.device("cuda:0")
    shape = KVShape("na", 6, 2, 64, tokens_per_block=16)
    NB, n = 96, 40
    kv_a, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="zeros")
    kv_b, _ = alloc_paged_cache(shape, NB, dev, "vllm", fill="zeros")
    reg_a, reg_b = register_tensors(kv_a, layout), register_tensors(kv_b, layout)
    chunk = reg_a.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    gen = torch.Generator().manual_seed(9)
    pool = torch.randint(0, 256, (NB, bb), dtype=torch.uint8, generator=gen).pin_memory()
    host = HostSide(pool.data_ptr(), shape.kv_dim * chunk, chunk, bb, NB)
    fn = _entry()
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream()
    rng = np.random.default_rng(2)
    for epoch in (1, 2):                                   # two calls in a row share the built-in array
        g = torch.from_numpy(rng.permutation(NB)[:n].astype(np.int64)).to(dev)
        c = torch.from_numpy(rng.permutation(NB)[:n].astype(np.int64)).to(dev)
        # ordinary entry point: scratch counters are a tensor the caller allocated
        flags_ref = torch.zeros(shape.num_layers, dtype=torch.int32, device=dev)
        status_ref = new_status(dev)
        scratch = torch.zeros(shape.num_layers, dtype=torch.int32, device=dev)
        p = make_params(reg_a, host, g, c, True, status_ptr=status_ref.data_ptr())
        p.update(done_counter_ptr=scratch.data_ptr(), dev_flags_ptr=flags_ref.data_ptr(), epoch=epoch, layer_major=1)
        _native.C.kv_copy(p, 6, 4096, 0, stream.cuda_stream)
        # the allocation-free entry point, through the C symbol
        flags = torch.zeros(shape.num_layers, dtype=torch.int32, device=dev)
        status = new_status(dev)
        a = _args(reg_b, host, g, c, flags, status, epoch, shape.num_layers)
        rc = fn(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream), err, len(err))
        assert rc == 0, err.value
        torch.cuda.synchronize()
        assert decode_status(status_ref) == 0 and decode_status(status) == 0
        assert flags.tolist() == [epoch] * shape.num_layers == flags_ref.tolist()
        assert int(scratch.abs().sum()) == 0               # the kernel leaves its counters at zero
        for ta, tb in zip(kv_a, kv_b):
            assert torch.equal(ta.view(torch.uint8), tb.view(torch.uint8))   # byte-identical (random bytes hold NaNs)
        gi = g
        want = pool[c.cpu()].view(n, shape.num_layers, shape.kv_dim, chunk)
        for l in range(shape.num_layers):
            got = kv_b[l][:, gi].contiguous().view(torch.uint8).reshape(shape.kv_dim, n, chunk).permute(1, 0, 2).cpu()
            assert torch.equal(got, want[:, l])


def test_noalloc_entry_rejects_sizes_beyond_its_array():
    fn = _entry()
    err = ctypes.create_string_buffer(256)
    dev = torch.device("cuda:0")
    shape = KVShape("na2", 2, 2, 64, tokens_per_block=16)
    kv, layout = alloc_paged_cache(shape, 8, dev, "vllm", fill="zeros")
    reg = register_tensors(kv, layout)
    host = HostSide(0, 0, 0, 0, 0)
    ids = torch.zeros(1, dtype=torch.int64, device=dev)
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    a = _args(reg, host, ids, ids, flags, new_status(dev), 1, 1025)      # one past FKV_NOALLOC_MAX_LAYERS
    rc = fn(ctypes.byref(a), None, err, len(err))
    assert rc != 0 and b"1024" in err.value
    torch.cuda.synchronize()


def test_noalloc_entry_rejects_a_short_tensor_table_and_releases_an_empty_call():
    fn = _entry()
    err = ctypes.create_string_buffer(256)
    dev = torch.device("cuda:0")
    shape = KVShape("na3", 4, 2, 64, tokens_per_block=16)
    kv, layout = alloc_paged_cache(shape, 8, dev, "vllm", fill="zeros")
    reg = register_tensors(kv, layout)
    chunk = reg.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    pool = torch.zeros(8, bb, dtype=torch.uint8).pin_memory()
    host = HostSide(pool.data_ptr(), shape.kv_dim * chunk, chunk, bb, 8)
    ids = torch.zeros(1, dtype=torch.int64, device=dev)
    flags = torch.zeros(shape.num_layers, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream()
    # a table one tensor short of what 4 layers address: refused on the host, nothing launched
    a = _args(reg, host, ids, ids, flags, new_status(dev), 1, shape.num_layers)
    a.num_gpu_ptrs = shape.num_layers - 1
    rc = fn(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream), err, len(err))
    assert rc == -1 and b"tensor table" in err.value
    torch.cuda.synchronize()
    assert flags.tolist() == [0] * shape.num_layers
    # an empty restore copies nothing and still publishes every layer's flag, in stream order
    empty = torch.zeros(0, dtype=torch.int64, device=dev)
    a = _args(reg, host, empty, empty, flags, new_status(dev), 7, shape.num_layers)
    rc = fn(ctypes.byref(a), ctypes.c_void_p(stream.cuda_stream), err, len(err))
    assert rc == 0, err.value
    torch.cuda.synchronize()
    assert flags.tolist() == [7] * shape.num_layers
