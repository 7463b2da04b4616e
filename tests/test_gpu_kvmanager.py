"""End-to-end on a GPU: KVManager put -> (clear) -> get with byte-exact checks,
over engine layouts, with the SSD tier, batches and the native transfer group."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config

pytestmark = pytest.mark.gpu


def _slots(blocks, T):
    return np.repeat(blocks, T) * T + np.tile(np.arange(T), len(blocks))


def _chunks(tensors, engine_layout, shape, blocks):
    """[n, L, K, chunk_bytes] uint8 copy of the given blocks."""
    idx = torch.as_tensor(blocks, device=tensors[0].device)
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


@pytest.mark.parametrize("engine_layout,shape", [
    ("vllm", KVShape("a", 4, 4, 64, tokens_per_block=16)),
    ("sglang", KVShape("b", 3, 2, 128, tokens_per_block=16)),
    ("trtllm", KVShape("c", 2, 2, 64, tokens_per_block=8)),
    ("vllm", KVShape("m", 5, 1, 576, use_mla=True, tokens_per_block=64)),
    # 288 tensors: more than the launch parameters carry, so the tensor table lives in device memory
    ("sglang", KVShape("deep", 144, 2, 16, tokens_per_block=8)),
])
def test_put_get_roundtrip(engine_layout, shape, tmp_path):
    dev = torch.device("cuda:0")
    T, NB = shape.tokens_per_block, 96
    kv, layout = alloc_paged_cache(shape, NB, dev, engine_layout, fill="normal", seed=11)
    cfg = CacheConfig(tokens_per_block=T, num_cpu_blocks=64, enable_ssd=True, num_ssd_blocks=256,
                      ssd_cache_dir=str(tmp_path))
    mgr = KVManager(make_model_config(shape), cfg)
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(120)
    try:
        rng = np.random.default_rng(5)
        n = 20
        tok = rng.integers(0, 50000, size=n * T + 3, dtype=np.int64)
        src = rng.permutation(NB)[:n].astype(np.int64)
        slot = np.concatenate([_slots(src, T), np.zeros(3, dtype=np.int64)])
        tid = mgr.put_async(tok, slot)
        rsp = mgr.wait(tid, completely=True)[tid]
        assert rsp.status.value == "success" and int(rsp.return_mask.sum()) == n * T
        want = _chunks(kv, engine_layout, shape, src)
        for t in kv:
            t.zero_()
        # host hit
        tid, mask = mgr.get_match(tok)
        assert int(mask.sum()) == n * T
        dst = rng.permutation(NB)[:n].astype(np.int64)
        mgr.launch(tid, _slots(dst, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        torch.cuda.synchronize()
        assert torch.equal(_chunks(kv, engine_layout, shape, dst), want)
        # SSD hit after the host tier was dropped
        mgr._clear_cpu_cache()
        for t in kv:
            t.zero_()
        tid, mask = mgr.get_match(tok)
        assert int(mask.sum()) == n * T
        dst2 = rng.permutation(NB)[:n].astype(np.int64)
        mgr.launch(tid, _slots(dst2, T))
        assert mgr.wait(tid)[tid].status.value == "success"
        torch.cuda.synchronize()
        assert torch.equal(_chunks(kv, engine_layout, shape, dst2), want)
        # a second put of the same tokens moves nothing
        tid = mgr.put_async(tok, slot)
        rsp = mgr.wait(tid, completely=True)[tid]
        assert rsp.status.value == "success" and int(rsp.return_mask.sum()) == 0
    finally:
        mgr.shutdown()


def test_batched_put_and_get_share_one_launch():
    dev = torch.device("cuda:0")
    shape = KVShape("a", 4, 2, 64, tokens_per_block=16)
    T, NB = 16, 200
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=12)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=128))
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(120)
    try:
        rng = np.random.default_rng(6)
        perm = rng.permutation(NB).astype(np.int64)
        reqs = []
        off = 0
        for n in (5, 9, 3, 12):
            reqs.append((rng.integers(0, 1000, size=n * T, dtype=np.int64), perm[off:off + n]))
            off += n
        ids = [mgr.put_match(t)[0] for t, _ in reqs]
        bid = mgr.launch(ids, [_slots(b, T) for _, b in reqs], as_batch=True)
        assert len(bid) == 1
        rsp = mgr.wait(bid, completely=True)[bid[0]]
        assert rsp.status.value == "success"
        assert [int(m.sum()) for m in rsp.return_mask] == [5 * T, 9 * T, 3 * T, 12 * T]
        want = [_chunks(kv, "vllm", shape, b) for _, b in reqs]
        for t in kv:
            t.zero_()
        ids = []
        for t, _ in reqs:
            tid, mask = mgr.get_match(t)
            assert int(mask.sum()) == len(t)
            ids.append(tid)
        dsts = [perm[100 + 20 * i:100 + 20 * i + len(b)] for i, (_, b) in enumerate(reqs)]
        bid = mgr.launch(ids, [_slots(d, T) for d in dsts], as_batch=True)
        assert mgr.wait(bid)[bid[0]].status.value == "success"
        torch.cuda.synchronize()
        for d, w in zip(dsts, want):
            assert torch.equal(_chunks(kv, "vllm", shape, d), w)
    finally:
        mgr.shutdown()
