"""Child process standing in for an engine worker: owns the paged KV cache on cuda:0, exports it
to the process that runs the data plane through CUDA IPC handles, and checks afterwards that the
bytes the manager moved landed where they should."""
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from flexkv_b200 import KVTPClient  # noqa: E402
from flexkv_b200.models import KVShape, alloc_paged_cache  # noqa: E402


def main() -> int:
    reg_ep, workdir = sys.argv[1], sys.argv[2]
    dev = torch.device("cuda", 0)
    shape = KVShape("ipc", 4, 4, 64, tokens_per_block=16)
    kv, layout = alloc_paged_cache(shape, 64, dev, "vllm", fill="normal", seed=11)
    vmm = None
    if len(sys.argv) > 3 and sys.argv[3] == "vmm":
        # the cache lives in ONE cuMemCreate allocation (a sleep-mode allocator's layout): no legacy IPC handle
        from flexkv_b200 import _native
        from flexkv_b200.common.memory_handle import DeviceSpan
        per = (kv[0].numel() * kv[0].element_size() + 255) // 256 * 256
        vmm = _native.C.vmm_alloc(per * len(kv), 0, False)
        span = torch.as_tensor(DeviceSpan(*vmm), device=dev)
        moved = []
        for i, t in enumerate(kv):
            m = span[i * per:i * per + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
            m.copy_(t)
            moved.append(m)
        kv = moved
        assert _native.C.vmm_is_vmm_pointer(kv[0].data_ptr())
    before = [t.clone() for t in kv]
    client = KVTPClient(reg_ep, dp_client_id=0, device_id=0, tp_rank=0)
    client.register_to_server(kv, layout)             # cuda_ipc handles: the consumer is another process
    open(os.path.join(workdir, "registered"), "w").close()
    t0 = time.time()
    while not os.path.exists(os.path.join(workdir, "moved")) and time.time() - t0 < 120:
        time.sleep(0.05)
    torch.cuda.synchronize()
    src, dst = [3, 9, 1, 30, 12], [40, 41, 42, 43, 44]
    ok = all(torch.equal(kv[l][:, dst], before[l][:, src]) for l in range(4))
    untouched = all(torch.equal(kv[l][:, 50:60], before[l][:, 50:60]) for l in range(4))
    with open(os.path.join(workdir, "result.json"), "w") as f:
        json.dump({"ok": bool(ok), "untouched": bool(untouched)}, f)
    while not os.path.exists(os.path.join(workdir, "exit")) and time.time() - t0 < 180:
        time.sleep(0.05)
    client.shutdown()
    if vmm is not None:
        from flexkv_b200 import _native
        from flexkv_b200.common.memory_handle import stop_fd_server
        stop_fd_server()
        del kv, before, span, moved, m
        torch.cuda.synchronize()
        _native.C.vmm_free(*vmm)
    return 0


if __name__ == "__main__":
    sys.exit(main())
