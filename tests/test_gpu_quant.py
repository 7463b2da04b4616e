"""Fused block-scaled FP8 offload against a plain PyTorch fp32 reference of the
same arithmetic: payload bytes and scales bit-exact, restored bf16 bit-exact to
the reference dequantisation, error bounded against the original."""
import numpy as np
import pytest
import torch

from flexkv_b200 import CacheConfig, KVManager
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config
from flexkv_b200.ops.kv_copy import HostSide, decode_status, new_status
from flexkv_b200.ops.kv_quant import kv_quant_fp8, packed_chunk_bytes, reference_pack, reference_unpack
from flexkv_b200.storage.gpu_layout import register_tensors

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [KVShape("q1", 3, 8, 128, tokens_per_block=16),       # 16384-element chunks, 2 tiles
                                   KVShape("q2", 2, 1, 576, use_mla=True, tokens_per_block=64),   # 36864: ragged last tile
                                   KVShape("q3", 2, 2, 64, tokens_per_block=8)])       # 1024-element chunks
def test_pack_unpack_match_reference(shape):
    dev = torch.device("cuda:0")
    NB, n = 40, 23
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=61)
    # widen the dynamic range and plant exact zeros so scale selection is exercised
    kv[0].mul_(37.0)
    kv[1].view(-1)[:4096].zero_()
    reg = register_tensors(kv, layout)
    E = reg.chunk_bytes // 2
    pc = packed_chunk_bytes(E)
    L, K = shape.num_layers, shape.kv_dim
    pool = torch.zeros(NB, L, K, pc, dtype=torch.uint8).pin_memory()
    host = HostSide(pool.data_ptr(), K * pc, pc, L * K * pc, NB)
    rng = np.random.default_rng(4)
    g = rng.permutation(NB)[:n].astype(np.int64)
    c = rng.permutation(NB)[:n].astype(np.int64)
    status = new_status(dev)
    keep = kv_quant_fp8(reg, host, g, c, h2d=False, num_ctas=7, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    gi = torch.from_numpy(g).to(dev)
    for l in range(L):
        for k in range(K):
            x = (kv[l][gi] if shape.use_mla else kv[l][k][gi]).reshape(n, E)
            want_q, want_s = reference_pack(x)
            got = pool[torch.from_numpy(c), l, k]
            assert torch.equal(got[:, :E], want_q.cpu()), (l, k)
            assert torch.equal(got[:, E:].contiguous().view(torch.float32), want_s.cpu()), (l, k)
    saved = [t.clone() for t in kv]
    for t in kv:
        t.zero_()
    g2 = rng.permutation(NB)[:n].astype(np.int64)
    keep += kv_quant_fp8(reg, host, g2, c, h2d=True, num_ctas=5, status=status)
    torch.cuda.synchronize()
    assert decode_status(status) == 0
    g2i = torch.from_numpy(g2).to(dev)
    for l in range(L):
        for k in range(K):
            orig = (saved[l][gi] if shape.use_mla else saved[l][k][gi]).reshape(n, E)
            q, s = reference_pack(orig)
            want = reference_unpack(q, s)
            got = (kv[l][g2i] if shape.use_mla else kv[l][k][g2i]).reshape(n, E)
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (l, k)
            # e4m3 keeps 3 mantissa bits: relative error of a group is bounded by 2^-4 of its amax
            err = (got.float() - orig.float()).abs().reshape(n, -1, 128).amax(-1)
            bound = orig.float().abs().reshape(n, -1, 128).amax(-1) / 16 + 1e-30
            assert bool((err <= bound).all())


def test_kvmanager_with_fp8_host_pool_halves_the_host_block():
    dev = torch.device("cuda:0")
    shape = KVShape("q4", 4, 8, 128, tokens_per_block=16)
    T, NB, n = 16, 64, 20
    kv, layout = alloc_paged_cache(shape, NB, dev, "vllm", fill="normal", seed=62)
    mgr = KVManager(make_model_config(shape), CacheConfig(tokens_per_block=T, num_cpu_blocks=48,
                                                          offload_quant="fp8_e4m3"))
    mgr.register_gpu_tensors(kv, layout)
    mgr.start()
    mgr.wait_ready(120)
    try:
        host = mgr.transfer_manager.storage.host
        assert host.block_bytes == shape.block_bytes // 2 + shape.block_bytes // 64
        rng = np.random.default_rng(8)
        tok = rng.integers(0, 1000, size=n * T, dtype=np.int64)
        src = rng.permutation(NB)[:n].astype(np.int64)
        slot = np.repeat(src, T) * T + np.tile(np.arange(T), n)
        tid = mgr.put_async(tok, slot)
        assert mgr.wait(tid, completely=True)[tid].status.value == "success"
        saved = [t.clone() for t in kv]
        for t in kv:
            t.zero_()
        dst = rng.permutation(NB)[:n].astype(np.int64)
        tid = mgr.get_async(tok, np.repeat(dst, T) * T + np.tile(np.arange(T), n))
        assert mgr.wait(tid)[tid].status.value == "success"
        torch.cuda.synchronize()
        si, di = torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev)
        for l in range(shape.num_layers):
            orig = saved[l][:, si].reshape(2, n, -1)
            q, s = reference_pack(orig)
            assert torch.equal(kv[l][:, di].reshape(2, n, -1).view(torch.int16), reference_unpack(q, s).view(torch.int16))
    finally:
        mgr.shutdown()
