"""Layerwise restore on a GPU: bytes, one eventfd unit per layer per restore and
none before the transfer, layer completion order, stream waits, device flags
with a bounded wait (reference: tests/test_layerwise_eventfd_timing.py:342-429)."""
import os
import struct

import numpy as np
import pytest
import torch

from flexkv_b200 import _native
from flexkv_b200.models import KVShape, alloc_paged_cache
from flexkv_b200.storage.gpu_layout import register_tensors

pytestmark = pytest.mark.gpu
C = _native.C


def _setup(shape, NB=128, notify="hostfunc", layers_per_batch=1, engine_layout="vllm"):
    dev = torch.device("cuda:0")
    kv, layout = alloc_paged_cache(shape, NB, dev, engine_layout, fill="normal", seed=21)
    reg = register_tensors(kv, layout)
    chunk = reg.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    pool = torch.zeros(NB, shape.num_layers, shape.kv_dim, chunk, dtype=torch.uint8).pin_memory()
    host = dict(base=pool.data_ptr(), layer_stride=shape.kv_dim * chunk, kv_stride=chunk, block_stride=bb,
                num_blocks=NB)
    opts = dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim, chunk_bytes=chunk, max_blocks_per_op=NB,
                notify_mode=notify, num_counters=3, layers_per_batch=layers_per_batch,
                h2d=dict(num_ctas=4, tile_bytes=8192, engine=0))
    grp = C.LayerwiseGroup([reg.as_native()], host, opts)
    xfer = C.TransferGroup([reg.as_native()], host, dict(num_layers=shape.num_layers, kv_dim=shape.kv_dim,
                                                         chunk_bytes=chunk, max_blocks_per_op=NB))
    return kv, reg, pool, grp, xfer


def _drain(fd):
    n = 0
    while True:
        try:
            n += struct.unpack("Q", os.read(fd, 8))[0]
        except BlockingIOError:
            return n


@pytest.mark.parametrize("notify,lpb", [("hostfunc", 1), ("polling", 1), ("flag", 1), ("hostfunc", 3), ("flag", 4),
                                        ("flag", 0), ("hostfunc", 0)])   # 0 = one launch, per-layer flags from the kernel
def test_restore_signals_each_layer_once(notify, lpb):
    shape = KVShape("lw", 6, 2, 64, tokens_per_block=16)
    kv, reg, pool, grp, xfer = _setup(shape, notify=notify, layers_per_batch=lpb)
    rng = np.random.default_rng(3)
    n = 40
    src = rng.permutation(128)[:n].astype(np.int64)
    cpu = rng.permutation(128)[:n].astype(np.int64)
    assert xfer.transfer(src, cpu, False, 0, shape.num_layers).status == 0
    want = [t[:, torch.from_numpy(src).cuda()].clone() for t in kv]
    for t in kv:
        t.zero_()
    for counter in (0, 2):
        fds = [grp.eventfd_of(counter, 0, l) for l in range(shape.num_layers)]
        assert all(_drain(fd) == 0 for fd in fds)                 # nothing before the transfer
        dst = rng.permutation(128)[:n].astype(np.int64)
        r = grp.restore(dst, cpu, counter)
        assert r.status == 0 and len(r.layer_done_ms) == shape.num_layers
        assert all(b >= a for a, b in zip(r.layer_done_ms, r.layer_done_ms[1:]))   # layers land in order
        assert [_drain(fd) for fd in fds] == [1] * shape.num_layers               # exactly one unit per layer
        other = [grp.eventfd_of(1, 0, l) for l in range(shape.num_layers)]
        assert all(_drain(fd) == 0 for fd in other)                                # other counters untouched
        d = torch.from_numpy(dst).cuda()
        for l in range(shape.num_layers):
            assert torch.equal(kv[l][:, d], want[l])
        # device and host flags carry the restore's epoch
        ep = grp.epoch_of(counter)
        flags = torch.empty(shape.num_layers, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        import ctypes
        host_flags = (ctypes.c_uint32 * shape.num_layers).from_address(grp.host_flags_ptr(0, counter))
        assert list(host_flags) == [ep] * shape.num_layers


def test_empty_restore_fires_every_layer_immediately():
    shape = KVShape("lw", 4, 2, 64, tokens_per_block=16)
    kv, reg, pool, grp, xfer = _setup(shape)
    e = np.zeros(0, dtype=np.int64)
    r = grp.restore(e, e, 1)
    assert r.status == 0
    assert [_drain(grp.eventfd_of(1, 0, l)) for l in range(4)] == [1, 1, 1, 1]


@pytest.mark.parametrize("lpb", [1, 0])
def test_model_stream_can_wait_per_layer_and_device_flags_release_consumers(lpb):
    shape = KVShape("lw", 5, 2, 128, tokens_per_block=16)
    kv, reg, pool, grp, xfer = _setup(shape, notify="flag", layers_per_batch=lpb)
    n = 64
    ids = np.arange(n, dtype=np.int64)
    assert xfer.transfer(ids, ids, False, 0, shape.num_layers).status == 0
    grp.restore(ids, ids, 0)                                       # first restore: epoch 1
    ep = grp.epoch_of(0)
    model = torch.cuda.Stream()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    starts = torch.zeros(shape.num_layers, dtype=torch.int64, device="cuda")
    # consumer kernels that wait (bounded) on the device flag of their layer, already satisfied by epoch `ep`
    for l in range(shape.num_layers):
        C.layer_stub(grp.device_flags_ptr(0, 0) + 4 * l, ep, 20_000, 500_000_000, status.data_ptr(),
                     starts.data_ptr() + 8 * l, 2, model.cuda_stream)
    model.synchronize()
    assert status.item() == 0 and bool((starts[1:] >= starts[:-1]).all())
    # stream-ordered wait on the per-layer event of a finished restore returns at once
    for l in range(shape.num_layers):
        grp.stream_wait_layer(0, 0, l, model.cuda_stream)
    model.synchronize()


def test_consumer_wait_runs_out_and_reports_status():
    """A flag that nothing sets: the wait gives up after its budget, sets the
    status word and the context stays usable."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.layer_stub(flag.data_ptr(), 5, 1000, 50_000_000, status.data_ptr(), 0, 1, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 1
    C.set_flags(flag.data_ptr(), 1, 7, torch.cuda.current_stream().cuda_stream)
    status.zero_()
    C.layer_stub(flag.data_ptr(), 5, 1000, 50_000_000, status.data_ptr(), 0, 1, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.item() == 0 and flag.item() == 7


@pytest.mark.parametrize("lpb", [0, 1])
def test_a_layer_flag_is_never_seen_before_the_layer_bytes(lpb):
    """Consumer kernels are launched BEFORE the restore, spin (bounded) on their layer's device flag and sum
    the layer's bytes the moment they see it: a flag published ahead of its data would give a stale sum."""
    shape = KVShape("lw", 6, 2, 128, tokens_per_block=16)
    NB = 128
    kv, reg, pool, grp, xfer = _setup(shape, NB=NB, notify="flag", layers_per_batch=lpb)
    ids = np.arange(NB, dtype=np.int64)
    assert xfer.transfer(ids, ids, False, 0, shape.num_layers).status == 0
    want = [int(t.view(torch.int64).sum().item()) & ((1 << 64) - 1) for t in kv]
    for rep in range(3):
        for t in kv:
            t.zero_()
        torch.cuda.synchronize()
        ep = grp.epoch_of(0) + 1                                   # the epoch the next restore on counter 0 publishes
        sums = torch.zeros(shape.num_layers, dtype=torch.int64, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        streams = [torch.cuda.Stream() for _ in range(shape.num_layers)]
        for l, s in enumerate(streams):                            # 6 layers x 2 CTAs: all resident at once
            C.layer_probe(grp.device_flags_ptr(0, 0) + 4 * l, ep, kv[l].data_ptr(), kv[l].numel() * 2, 2_000_000_000,
                          status.data_ptr(), sums.data_ptr() + 8 * l, 2, s.cuda_stream)
        r = grp.restore(ids, ids, 0)
        assert r.status == 0
        torch.cuda.synchronize()
        assert status.item() == 0
        got = [int(v) & ((1 << 64) - 1) for v in sums.tolist()]
        assert got == want, (rep, lpb)


@pytest.mark.parametrize("lpb", [1, 0])
def test_consumer_waits_bind_to_the_reserved_epoch_not_to_the_previous_restore(lpb):
    """The model thread reserves the epoch before the restore is issued, waits on the host until the restore's
    launches are queued, then queues its per-layer stream waits: they bind to THIS restore, not to the previous
    one's flags (which already hold an older epoch)."""
    import threading
    shape = KVShape("lw", 5, 2, 128, tokens_per_block=16)
    kv, reg, pool, grp, xfer = _setup(shape, notify="flag", layers_per_batch=lpb)
    n = 64
    ids = np.arange(n, dtype=np.int64)
    assert xfer.transfer(ids, ids, False, 0, shape.num_layers).status == 0
    want = [t[:, :n].clone() for t in kv]
    assert grp.restore(ids, ids, 0).status == 0              # a first restore: the flags hold epoch 1
    for t in kv:
        t.zero_()
    model = torch.cuda.Stream()
    ep = grp.begin_restore(0)
    assert ep == grp.epoch_of(0) == 2
    snaps = []
    assert not grp.wait_launched(0, ep, 50)                   # nothing queued yet for this epoch
    th = threading.Thread(target=lambda: grp.restore(ids, ids, 0))
    th.start()
    assert grp.wait_launched(0, ep, 10000)
    with torch.cuda.stream(model):
        for l in range(shape.num_layers):
            grp.stream_wait_layer(0, 0, l, model.cuda_stream, ep)
            snaps.append(kv[l][:, :n].clone())                # what the model would read once released
    th.join()
    model.synchronize()
    assert grp.epoch_of(0) == 2 and grp.counter_status(0) == 0
    for l in range(shape.num_layers):
        assert torch.equal(snaps[l], want[l]), l


def test_failed_disk_stage_releases_every_waiter_with_the_failure_signal(tmp_path):
    """The failure is made on the host (an injected EIO in the SSD engine). Nothing is copied, the result and
    counter_status carry the error, every layer's eventfd fires and a stream parked on a layer flag is released."""
    shape = KVShape("lw", 4, 2, 64, tokens_per_block=16)
    kv, reg, pool, grp, xfer = _setup(shape, notify="flag", layers_per_batch=0)
    chunk = reg.chunk_bytes
    bb = shape.num_layers * shape.kv_dim * chunk
    paths = [[str(tmp_path / "blk.bin")]]
    ssd = C.SsdIoEngine(paths, bb, 16, create=True, try_direct=False, iouring_entries=0, num_threads=2)
    lay = dict(cpu_layer_stride=shape.kv_dim * chunk, cpu_kv_stride=chunk, cpu_block_stride=bb,
               ssd_layer_stride=shape.kv_dim * chunk, ssd_kv_stride=chunk, ssd_block_stride=bb, chunk_bytes=chunk,
               num_layers=shape.num_layers, kv_dim=shape.kv_dim, block_first=True)
    ids = np.arange(4, dtype=np.int64)
    ssd.set_fault(3, 0)                                       # every IO fails
    model = torch.cuda.Stream()
    ep = grp.begin_restore(1)
    before = [t.clone() for t in kv]
    r = grp.restore(ids, ids, 1, ssd, lay, ids, ids)
    assert r.status != 0 and r.epoch == ep
    assert grp.counter_status(1) != 0 and grp.wait_launched(1, ep, 1000)      # a failed restore counts as queued
    for l in range(shape.num_layers):
        grp.stream_wait_layer(0, 1, l, model.cuda_stream, ep)
    model.synchronize()                                       # the flags were released from the host: no hang
    # every layer's eventfd fired once: an engine hook blocked on it wakes up and reads the failure
    # from counter_status() / the failed task
    assert [_drain(grp.eventfd_of(1, 0, l)) for l in range(shape.num_layers)] == [1] * shape.num_layers
    for a, b in zip(before, kv):
        assert torch.equal(a, b)                              # nothing was copied
    ssd.set_fault(0, 0)
    r = grp.restore(ids, ids, 1, ssd, lay, ids, ids)          # the next restore on the counter is clean again
    assert r.status == 0 and grp.counter_status(1) == 0
    assert [_drain(grp.eventfd_of(1, 0, l)) for l in range(shape.num_layers)] == [1] * shape.num_layers


@pytest.mark.parametrize("lpb", [0, 2])
def test_layerwise_restore_from_a_packed_host_pool(lpb):
    """Host pool in the lossless codec's packed form: the restore unpacks layer by layer (one fused launch
    with per-layer flags, or one launch per layer batch), signals every layer once and is bit-exact."""
    from flexkv_b200.ops.kv_compress import chunk_slot_bytes, kv_compress, size_table_entries
    from flexkv_b200.ops.kv_copy import HostSide, decode_status, new_status
    dev = torch.device("cuda:0")
    shape = KVShape("lwc", 4, 8, 128, tokens_per_block=16)           # 16384-element chunks, two tiles each
    NB, n = 64, 24
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=33)
    reg = register_tensors(kv, layout)
    E = reg.chunk_bytes // 2
    L, K = shape.num_layers, shape.kv_dim
    slot = chunk_slot_bytes(E)
    pool = torch.zeros(NB, L, K, slot, dtype=torch.uint8).pin_memory()
    table = torch.zeros(size_table_entries(NB, L, K, E), dtype=torch.int32).pin_memory()
    host = HostSide(pool.data_ptr(), K * slot, slot, L * K * slot, NB)
    rng = np.random.default_rng(4)
    src = rng.permutation(NB)[:n].astype(np.int64)
    cpu = rng.permutation(NB)[:n].astype(np.int64)
    status = new_status(dev)
    keep = kv_compress(reg, host, table, src, cpu, h2d=False, num_ctas=6, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    want = [t[:, torch.from_numpy(src).cuda()].clone() for t in kv]
    for t in kv:
        t.zero_()
    opts = dict(num_layers=L, kv_dim=K, chunk_bytes=reg.chunk_bytes, max_blocks_per_op=NB, notify_mode="flag",
                num_counters=2, layers_per_batch=lpb, size_table_ptr=table.data_ptr(), size_table_layers=L,
                codec_pipelines=6)
    grp = C.LayerwiseGroup([reg.as_native()], dict(base=pool.data_ptr(), layer_stride=K * slot, kv_stride=slot,
                                                    block_stride=L * K * slot, num_blocks=NB), opts)
    dst = rng.permutation(NB)[:n].astype(np.int64)
    r = grp.restore(dst, cpu, 1)
    assert r.status == 0 and grp.counter_status(1) == 0
    assert [_drain(grp.eventfd_of(1, 0, l)) for l in range(L)] == [1] * L
    d = torch.from_numpy(dst).cuda()
    for l in range(L):
        assert torch.equal(kv[l][:, d].view(torch.int16), want[l].view(torch.int16)), l
    del keep
