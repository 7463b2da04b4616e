"""GPU batched block keys against the host hasher (which is itself pinned to canonical XXH64
vectors in test_hash.py): ragged batches, namespaces, block sizes that do and do not align with
the 32-byte stripes."""
import numpy as np
import pytest
import torch

from flexkv_b200.common.block import hash_blocks
from flexkv_b200.ops.kv_hash import gpu_block_hashes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tpb", [1, 3, 4, 16, 64])
@pytest.mark.parametrize("namespace", [None, ["lora-7"], ["tenant", "a", "salt123"]])
def test_matches_host_hasher(tpb, namespace):
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(tpb)
    lens = [0, 1, 2, 5, 31, 64, 257, 1000, 8192, 4099]
    seqs = [rng.integers(-2**62, 2**62, size=n, dtype=np.int64) for n in lens]
    got = gpu_block_hashes([torch.from_numpy(s).to(dev) for s in seqs], tpb, namespace)
    torch.cuda.synchronize()
    for s, g in zip(seqs, got):
        want = hash_blocks(s, tpb, namespace)
        assert g.cpu().numpy().view(np.uint64).tolist() == want.tolist()


def test_large_batch_is_consistent():
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 128256, size=2048, dtype=np.int64) for _ in range(300)]
    got = gpu_block_hashes([torch.from_numpy(s).to(dev) for s in seqs], 16)
    torch.cuda.synchronize()
    for i in (0, 1, 150, 299):
        assert got[i].cpu().numpy().view(np.uint64).tolist() == hash_blocks(seqs[i], 16).tolist()
