"""torchrun worker: NVSwitch fan-out restore. Rank 0 reads host blocks once and
multimem-stores them into every rank's symmetric KV cache; all ranks verify the
bytes. Teardown is orderly on every path (barrier, then destroy) because a rank
that leaves while its memory is bound to a multicast object disturbs the others."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    result = {"rank": rank, "ok": False}
    try:
        from flexkv_b200.common.storage import KVCacheLayout, KVCacheLayoutType
        from flexkv_b200.ops.kv_copy import HostSide, decode_status, new_status
        from flexkv_b200.parallel.nvls import alloc_symmetric_kv_layers, fanout_restore, wait_flag
        from flexkv_b200.storage.gpu_layout import register_tensors

        # MLA-shaped latent cache, identical on every rank: L layers of [N, T, 576] bf16
        L, N, T, D = 4, 64, 64, 576
        per_layer = N * T * D * 2
        try:
            # two symmetric segments of two layers each: the kernel reaches every tensor through the
            # multicast mapping of the segment that holds it
            sym = alloc_symmetric_kv_layers(L, per_layer, dev, segment_bytes=2 * per_layer)
        except RuntimeError as e:
            result.update(ok=True, skipped=str(e))
            return 0
        assert len(sym.segments) == 2
        kv = [sym.layer_tensor(l, (N, T, D), torch.bfloat16) for l in range(L)]
        layout = KVCacheLayout(KVCacheLayoutType.LAYERFIRST, L, N, T, 1, D, is_mla=True)
        reg = register_tensors(kv, layout)
        chunk = reg.chunk_bytes
        n = 24
        g = torch.Generator().manual_seed(5)
        pool = torch.randint(0, 256, (N, L, 1, chunk), dtype=torch.uint8, generator=g).pin_memory()
        host = HostSide(pool.data_ptr(), chunk, chunk, L * chunk, N)
        rng = np.random.default_rng(1)
        gpu_blocks = rng.permutation(N)[:n].astype(np.int64)
        cpu_blocks = rng.permutation(N)[:n].astype(np.int64)
        status = new_status(dev)
        scratch = torch.zeros(1, dtype=torch.int32, device=dev)
        timings = []
        for epoch in (1, 2, 3):
            for t in kv:
                t.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if rank == 0:
                e0.record()
                keep = fanout_restore(sym, reg, host, gpu_blocks, cpu_blocks, epoch, scratch, status)
                e1.record()
                torch.cuda.synchronize()
                timings.append(e0.elapsed_time(e1))
                assert decode_status(status) == 0, decode_status(status)
            assert wait_flag(sym, epoch, timeout_s=10.0), "completion flag never arrived"
            torch.cuda.synchronize()
            for l in range(L):
                got = kv[l][torch.from_numpy(gpu_blocks).to(dev)].contiguous().view(torch.uint8).reshape(n, -1).cpu()
                want = pool[torch.from_numpy(cpu_blocks), l, 0]
                assert torch.equal(got, want), f"rank {rank} layer {l} differs"
            untouched = np.setdiff1d(np.arange(N), gpu_blocks)
            assert int(kv[0][torch.from_numpy(untouched).to(dev)].abs().sum()) == 0
            dist.barrier()
        # the same kernel behind the public API: rank 0's manager restores a prefix into every rank's cache
        from flexkv_b200.utils import selfcheck
        mgr_ok = selfcheck.nvls_manager_restore_all_ranks(dev, rank, world)
        result.update(ok=mgr_ok is True, manager_path=mgr_ok, ms=timings, bytes=n * L * chunk,
                      why=selfcheck.last_failure)
        return 0
    except Exception as e:  # noqa: BLE001
        result["error"] = repr(e)
        return 1
    finally:
        out = os.environ.get("FKV_RESULT_DIR")
        if out:
            with open(os.path.join(out, f"nvls_rank{rank}.json"), "w") as f:
                json.dump(result, f)
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
