"""Child process: the second node of a two-node tensor-parallel group. Holds rank 1's
paged cache (host stand-in tensors), serves the master's graphs, and on shutdown writes
what it holds so the parent can check the bytes."""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from flexkv_b200 import CacheConfig  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache, make_model_config  # noqa: E402
from flexkv_b200.storage.gpu_layout import register_tensors  # noqa: E402
from flexkv_b200.transfer_manager import TransferManagerOnRemote  # noqa: E402


def main() -> int:
    cmd, res, qry, out = sys.argv[1:5]
    register_port = sys.argv[5] if len(sys.argv) > 5 else None      # this node's ranks send their page lists here
    T = 4
    shape = KVShape("mn", 2, 4, 16, tokens_per_block=T)
    mc = make_model_config(shape, tp_size=2, nnodes=2)
    cc = CacheConfig(tokens_per_block=T, num_cpu_blocks=24)
    node = TransferManagerOnRemote(mc, cc, cmd, res, qry, require_gpu=True, gpu_register_port=register_port)
    kv, layout = alloc_paged_cache(shape, 64, "cpu", "vllm", tp_size=2, fill="normal", seed=77)
    before = [t.clone() for t in kv]
    node.register_gpu(register_tensors(kv, layout, tp_rank=1))
    node.serve_forever()
    torch.save({"before": before, "after": kv}, out)
    print(json.dumps({"ok": True}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
