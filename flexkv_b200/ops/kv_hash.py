"""Batched block keys on the GPU (``csrc/kernels/kv_hash.cu``): cumulative streaming XXH64 over
int64 token ids, bit-identical to the host hasher. Worth it for token ids that already live on
the device or for thousands of long sequences at once; a single request is faster on the host."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import _native
from ..common.block import namespace_prefix


def gpu_block_hashes(seqs: Sequence[torch.Tensor], tokens_per_block: int, namespace: Optional[List[str]] = None,
                     stream: Optional[torch.cuda.Stream] = None) -> List[torch.Tensor]:
    """``seqs``: int64 CUDA tensors (one per sequence, same device). Returns one uint64-valued
    int64 CUDA tensor of block keys per sequence (view with ``.view(torch.uint64)`` or copy to numpy)."""
    if not seqs:
        return []
    dev = seqs[0].device
    lens = [int(s.numel()) for s in seqs]
    flat = torch.cat([s.reshape(-1) for s in seqs]) if len(seqs) > 1 else seqs[0].reshape(-1).contiguous()
    offs = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64, device=dev)
    nblk = [n // tokens_per_block for n in lens]
    ooffs = torch.tensor(np.concatenate([[0], np.cumsum(nblk)]), dtype=torch.int64, device=dev)
    out = torch.empty(max(1, sum(nblk)), dtype=torch.int64, device=dev)
    ns = namespace_prefix(namespace)
    ns_t = torch.from_numpy(np.ascontiguousarray(ns, dtype=np.int64)).to(dev) if ns is not None and len(ns) else None
    s = stream if stream is not None else torch.cuda.current_stream(dev)
    _native.C.kv_block_hashes(flat.data_ptr(), offs.data_ptr(), len(seqs), int(tokens_per_block),
                              ns_t.data_ptr() if ns_t is not None else 0, int(ns_t.numel()) if ns_t is not None else 0,
                              out.data_ptr(), ooffs.data_ptr(), s.cuda_stream)
    res, o = [], 0
    for n in nblk:
        res.append(out[o:o + n])
        o += n
    # keep inputs alive until the launch has been ordered on the stream
    flat.record_stream(s)
    return res
