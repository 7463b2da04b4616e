#!/usr/bin/env python
"""Block-key generation: host hasher (one core, and batched over 8 threads) against the GPU kernel
with token ids already resident on the device. 8K-token sequences, 16-token blocks. CUDA events
for the kernel (launch overhead of the Python wrapper excluded and included)."""
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200 import _native  # noqa: E402
from flexkv_b200.ops.kv_hash import gpu_block_hashes  # noqa: E402

C = _native.C


def main() -> None:
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(0)
    for nseq in (1, 64, 1024, 8192):
        seqs = [rng.integers(0, 128256, size=8192, dtype=np.int64) for _ in range(min(nseq, 1024))]
        seqs = (seqs * ((nseq + len(seqs) - 1) // len(seqs)))[:nseq]
        t0 = time.perf_counter()
        for s in seqs[:256]:
            C.gen_hashes(s, 16, None)
        host_one = (time.perf_counter() - t0) / min(nseq, 256)
        t0 = time.perf_counter()
        C.gen_hashes_batch(seqs, 16, None, 8)
        host_batch = (time.perf_counter() - t0) / nseq
        flat = torch.from_numpy(np.concatenate(seqs)).to(dev)
        offs = torch.arange(0, (nseq + 1) * 8192, 8192, dtype=torch.int64, device=dev)
        ooffs = torch.arange(0, (nseq + 1) * 512, 512, dtype=torch.int64, device=dev)
        out = torch.empty(nseq * 512, dtype=torch.int64, device=dev)
        ms = []
        for i in range(8):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            C.kv_block_hashes(flat.data_ptr(), offs.data_ptr(), nseq, 16, 0, 0, out.data_ptr(), ooffs.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ms.append(e0.elapsed_time(e1))
        k = float(np.median(ms))
        want = C.gen_hashes(seqs[-1], 16, None)
        assert out[-512:].cpu().numpy().view(np.uint64).tolist() == want.tolist()
        t0 = time.perf_counter()
        r = gpu_block_hashes([flat[i * 8192:(i + 1) * 8192] for i in range(min(nseq, 64))], 16)
        torch.cuda.synchronize()
        wrap = (time.perf_counter() - t0) / min(nseq, 64)
        print(json.dumps(dict(sequences=nseq, tokens_each=8192, host_us_per_seq=round(host_one * 1e6, 1),
                              host_batched_us_per_seq=round(host_batch * 1e6, 1), gpu_kernel_ms=round(k, 3),
                              gpu_us_per_seq=round(k * 1e3 / nseq, 2),
                              gpu_gtokens_per_s=round(nseq * 8192 / k / 1e6, 2),
                              wrapper_us_per_seq_incl_launch=round(wrap * 1e6, 1))), flush=True)


if __name__ == "__main__":
    main()
