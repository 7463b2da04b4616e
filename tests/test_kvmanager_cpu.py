"""KVManager end to end without a GPU: the engine's paged cache is a host
tensor, the data plane runs on CPU threads with the kernels' addressing, the SSD
tier is real files. Deterministic fill, byte-exact checks (reference:
tests/test_kvmanager.py, tests/test_reset_cache.py, tests/test_namespace_isolation.py)."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config


def slots(blocks, T):
    return np.repeat(np.asarray(blocks, dtype=np.int64), T) * T + np.tile(np.arange(T), len(blocks))


def chunks(tensors, engine_layout, shape, blocks):
    idx = torch.as_tensor(np.asarray(blocks))
    out = []
    for l in range(shape.num_layers):
        per_kv = []
        for k in range(shape.kv_dim):
            if engine_layout == "vllm":
                t = tensors[l][idx] if shape.use_mla else tensors[l][k][idx]
            elif engine_layout == "sglang":
                t = tensors[k * shape.num_layers + l][idx] if shape.kv_dim == 2 else tensors[l][idx]
            else:
                t = tensors[0][idx, l, k]
            per_kv.append(t.contiguous().view(torch.uint8).reshape(len(blocks), -1))
        out.append(torch.stack(per_kv, 1))
    return torch.stack(out, 1)


def start(shape, engine_layout, NB=64, tp=1, **cache_kw):
    mgr = KVManager(make_model_config(shape, tp_size=tp), CacheConfig(tokens_per_block=shape.tokens_per_block,
                                                                      **cache_kw), require_gpu=True)
    caches = []
    for r in range(tp):
        kv, layout = alloc_paged_cache(shape, NB, "cpu", engine_layout, tp_size=tp, fill="normal", seed=100 + r)
        mgr.register_gpu_tensors(kv, layout, tp_rank=r)
        caches.append(kv)
    mgr.start()
    mgr.wait_ready(60)
    return mgr, caches


@pytest.mark.parametrize("engine_layout,shape", [
    ("vllm", KVShape("a", 3, 4, 16, tokens_per_block=4)),
    ("sglang", KVShape("b", 2, 2, 32, tokens_per_block=8)),
    ("trtllm", KVShape("c", 2, 2, 16, tokens_per_block=4)),
    ("vllm", KVShape("m", 3, 1, 64, use_mla=True, tokens_per_block=4)),
    ("sglang", KVShape("deep", 130, 2, 8, tokens_per_block=4)),      # 260 tensors: past the inline pointer table
])
def test_roundtrip_host_and_ssd(engine_layout, shape, tmp_path):
    T = shape.tokens_per_block
    mgr, (kv,) = start(shape, engine_layout, num_cpu_blocks=32, enable_ssd=True, num_ssd_blocks=128,
                       ssd_cache_dir=str(tmp_path))
    try:
        rng = np.random.default_rng(0)
        tok = rng.integers(0, 1000, size=9 * T + 1, dtype=np.int64)
        src = rng.permutation(64)[:9]
        tid = mgr.put_async(tok, np.concatenate([slots(src, T), [0]]))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        want = chunks(kv, engine_layout, shape, src)
        for t in kv:
            t.zero_()
        tid, mask = mgr.get_match(tok)
        assert mask.sum() == 9 * T
        dst = rng.permutation(64)[:9]
        mgr.launch(tid, slots(dst, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        assert torch.equal(chunks(kv, engine_layout, shape, dst), want)
        mgr._clear_cpu_cache()
        for t in kv:
            t.zero_()
        tid = mgr.get_async(tok, np.concatenate([slots(dst, T), [0]]))
        r = mgr.wait(tid)[tid]
        assert r.status.value == "success" and r.return_mask.sum() == 9 * T
        assert torch.equal(chunks(kv, engine_layout, shape, dst), want)
    finally:
        mgr.shutdown()


def test_tensor_parallel_ranks_share_one_host_block():
    shape = KVShape("tp", 2, 4, 16, tokens_per_block=4)
    T = 4
    mgr, caches = start(shape, "vllm", tp=2, num_cpu_blocks=16)
    try:
        tok = np.arange(5 * T, dtype=np.int64)
        src = np.array([3, 9, 1, 30, 12])
        tid = mgr.put_async(tok, slots(src, T))
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        rank_shape = KVShape("r", 2, 2, 16, tokens_per_block=4)        # heads per rank
        want = [chunks(kv, "vllm", rank_shape, src) for kv in caches]
        # host block = [rank][layer][kv][chunk]: rank r starts at r * block_bytes / tp
        host = mgr.transfer_manager.storage.host
        from flexkv_b200.common.block import SequenceMeta
        cpu_ids = mgr.kv_task_engine.cache_engine.cpu_cache_engine.match(SequenceMeta(tok, T)).physical_blocks
        for r in range(2):
            for i, b in enumerate(cpu_ids):
                blk = torch.from_numpy(host.block_view(int(b)).copy())
                half = blk.numel() // 2
                assert torch.equal(blk[r * half:(r + 1) * half], want[r][i].reshape(-1))
        for kv in caches:
            for t in kv:
                t.zero_()
        dst = np.array([7, 8, 40, 41, 2])
        tid = mgr.get_async(tok, slots(dst, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        for r in range(2):
            assert torch.equal(chunks(caches[r], "vllm", rank_shape, dst), want[r])
    finally:
        mgr.shutdown()


def test_eviction_keeps_serving_and_namespaces_isolate():
    shape = KVShape("e", 2, 2, 16, tokens_per_block=4)
    T = 4
    mgr, (kv,) = start(shape, "vllm", num_cpu_blocks=12)
    try:
        seqs = [np.arange(1000 * i, 1000 * i + 5 * T, dtype=np.int64) for i in range(4)]
        for i, s in enumerate(seqs):
            tid = mgr.put_async(s, slots(range(5 * i, 5 * i + 5), T))
            assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        probes = [mgr.get_match(s) for s in seqs]
        hits = [int(m.sum()) for _, m in probes]
        mgr.cancel([t for t, _ in probes])          # matched-but-unlaunched gets pin their nodes
        assert hits[-1] == 5 * T and hits[-2] == 5 * T and hits[0] == 0       # LRU: oldest went first
        assert sum(hits) <= 12 * T
        tid = mgr.put_async(seqs[3], slots(range(5), T), namespace=["tenant-a"])
        assert mgr.wait(tid, completely=True)[tid].return_mask.sum() == 5 * T   # other namespace: stored again
        assert mgr.get_match(seqs[3], namespace=["tenant-b"])[1].sum() == 0
        mgr.reset()
        assert all(int(mgr.get_match(s)[1].sum()) == 0 for s in seqs)
    finally:
        mgr.shutdown()


def test_injected_worker_failure_surfaces_as_failed():
    shape = KVShape("f", 2, 2, 16, tokens_per_block=4)
    T = 4
    mgr, (kv,) = start(shape, "vllm", num_cpu_blocks=16)
    try:
        from flexkv_b200.common.transfer import TransferType, WorkerKey
        w = mgr.transfer_manager.engine.worker_for(WorkerKey(0, 0), TransferType.D2H)
        w.fail_next = 1
        tok = np.arange(5 * T, dtype=np.int64)
        tid = mgr.put_async(tok, slots(range(5), T))
        assert mgr.wait(tid, timeout=5, completely=True)[tid].status.value == "failed"
        assert mgr.get_match(tok)[1].sum() == 0
        tid = mgr.put_async(tok, slots(range(5), T))                          # the next attempt works
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        assert mgr.get_match(tok)[1].sum() == 5 * T
    finally:
        mgr.shutdown()


def test_shutdown_lets_go_of_imported_cache_mappings():
    """A cache opened from another process's handle is closed when the manager shuts down: its owner may free
    it right afterwards (freeing exported memory that an importer still maps is undefined in CUDA)."""
    shape = KVShape("a", 2, 2, 16, tokens_per_block=4)
    mgr, (kv,) = start(shape, "vllm", num_cpu_blocks=16)
    closed = []

    class Handle:
        def close(self):
            closed.append(id(self))

    h = [Handle(), Handle()]
    reg = next(iter(mgr.transfer_manager.storage.gpu_regs.values()))[0]
    reg.keepalive = h + [h[0]]                       # the same handle listed twice is closed once
    mgr.shutdown()
    assert sorted(closed) == sorted(id(x) for x in h)


def test_multicast_registration_stands_for_its_whole_tp_group():
    """One registration that carries multicast addresses counts as every rank of a shared-KV tensor-parallel
    group when the data plane waits for its registrations."""
    from flexkv_b200.storage.gpu_layout import register_tensors
    from flexkv_b200.transfer_manager import TransferManager
    shape = KVShape("m", 2, 1, 64, use_mla=True, tokens_per_block=4)
    tm = TransferManager(make_model_config(shape, tp_size=4), CacheConfig(tokens_per_block=4, num_cpu_blocks=8),
                         require_gpu=True)
    kv, layout = alloc_paged_cache(shape, 8, "cpu", "vllm")
    reg = register_tensors(kv, layout)
    tm.register_gpu(reg)
    assert tm._expected_registrations() == 4 and tm._registrations_arrived() == 1
    reg.mc_ptrs = [int(p) for p in reg.ptrs]
    reg.mc_flag_ptr = 1
    assert tm._registrations_arrived() == 4


def test_a_rank_named_by_the_references_flat_id_lands_on_its_stage_local_rank():
    """``KVTPClient(..., pp_rank=1, intra_client_id=pp_rank * ranks_per_stage + rank)`` as the reference's adapters
    call it: the data plane keeps the rank inside the stage."""
    from flexkv_b200.storage.gpu_layout import GpuRegistration
    from flexkv_b200.transfer_manager import TransferManager
    tm = TransferManager.__new__(TransferManager)
    import threading
    tm._reg_cv = threading.Condition()
    tm._pending_regs = []
    tm.model_config = make_model_config(KVShape("x", 4, 4, 16, tokens_per_block=4), tp_size=2, pp_size=2)
    for pp, flat, want in ((0, 1, 1), (1, 2, 0), (1, 3, 1), (1, 1, 1)):
        reg = GpuRegistration.__new__(GpuRegistration)
        reg.pp_rank, reg.tp_rank = pp, flat
        tm.register_gpu(reg)
        assert tm._pending_regs[-1].tp_rank == want, (pp, flat)
