"""Run analysis and routing of the copy-engine path (reference behaviour:
csrc/ce_transfer.cu:37-104 segments contiguous (gpu, cpu) id runs and picks a path)."""
import numpy as np

from flexkv_b200 import _native

C = _native.C


def _params(g, c, *, layers=4, kv=2, chunk=32768, gpu_blockfirst=False, NB=4096):
    g = np.ascontiguousarray(g, dtype=np.int64)
    c = np.ascontiguousarray(c, dtype=np.int64)
    block = layers * kv * chunk
    d = dict(gpu_ptrs=[0x1000000] if gpu_blockfirst else [0x1000000 + i * NB * kv * chunk for i in range(layers)],
             idx_layer_mul=0 if gpu_blockfirst else 1, idx_kv_mul=0,
             g_layer_stride=kv * chunk if gpu_blockfirst else 0,
             g_kv_stride=chunk if gpu_blockfirst else NB * chunk,
             g_block_stride=block if gpu_blockfirst else chunk,
             cpu_base=0x7f0000000000, c_layer_stride=kv * chunk, c_kv_stride=chunk, c_block_stride=block,
             gpu_blocks_ptr=g.ctypes.data, cpu_blocks_ptr=c.ctypes.data, num_pairs=len(g), layer_start=0,
             num_layers=layers, kv_dim=kv, chunk_bytes=chunk, gpu_num_blocks=NB, cpu_num_blocks=NB)
    return d, (g, c)


def test_runs_split_where_either_side_jumps():
    g = [10, 11, 12, 20, 21, 30]
    c = [5, 6, 7, 8, 100, 101]
    d, keep = _params(g, c)
    runs, path, copies, status = C.ce_plan(d, 1 << 30, 0)
    assert runs.tolist() == [[10, 5, 3], [20, 8, 1], [21, 100, 1], [30, 101, 1]]
    assert status == 0
    assert path == "segment_2d" and copies == 4 * 4 * 2


def test_long_run_layerfirst_gpu_goes_2d_and_blockfirst_goes_contiguous():
    n = 512
    d, keep = _params(np.arange(n) + 7, np.arange(n) + 99)
    runs, path, copies, _ = C.ce_plan(d)
    assert runs.tolist() == [[7, 99, n]] and path == "segment_2d" and copies == 8      # 16 MiB per copy
    d, keep = _params(np.arange(64) + 7, np.arange(64) + 99)
    assert C.ce_plan(d)[1] == "kernel"                                                  # 2 MiB per copy: not worth it
    d, keep = _params(np.arange(n) + 7, np.arange(n) + 99, gpu_blockfirst=True)
    runs, path, copies, _ = C.ce_plan(d)
    assert path == "contig_blocks" and copies == 1


def test_scattered_ids_stay_on_the_kernel():
    rng = np.random.default_rng(0)
    g = rng.permutation(4096)[:512]
    c = rng.permutation(4096)[:512]
    d, keep = _params(g, c)
    runs, path, copies, _ = C.ce_plan(d)
    assert path == "kernel" and copies == 0 and len(runs) > 400
    # a layer sub-range of a block-first cache is not one span per run
    d, keep = _params(np.arange(64), np.arange(64), gpu_blockfirst=True)
    d["num_layers"] = 2
    assert C.ce_plan(d, 1 << 30, 0)[1] == "segment_2d"


def test_out_of_range_ids_are_dropped_and_flagged():
    d, keep = _params([1, 2, 5000, 3], [1, 2, 3, -4], NB=4096)
    runs, path, copies, status = C.ce_plan(d, 1 << 30, 0)
    assert runs.tolist() == [[1, 1, 2]]
    assert status == 1 | 2      # gpu and cpu range bits
