"""Child process that maps two tensors of another process's cuMemCreate allocation through their
handles, checks what the owner wrote, writes back and unmaps."""
import os
import pickle
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from flexkv_b200.common import memory_handle as mh  # noqa: E402


def main() -> int:
    with open(sys.argv[1], "rb") as f:
        ha, hb = pickle.load(f)
    torch.cuda.set_device(0)
    pa, pb = ha.open(), hb.open()
    assert pb - pa == hb.vmm_offset - ha.vmm_offset          # one mapping serves both tensors
    a = torch.as_tensor(mh.DeviceSpan(pa, ha.nbytes), device="cuda:0").view(torch.bfloat16).view(*ha.shape)
    b = torch.as_tensor(mh.DeviceSpan(pb, hb.nbytes), device="cuda:0").view(torch.int32)
    want = torch.arange(512 * 1024, device="cuda:0").remainder(251).to(torch.bfloat16).view(512, 1024)
    ok = bool(torch.equal(a, want)) and bool((b == 7).all())
    b.fill_(9)
    a[3, 5] = -1.0
    torch.cuda.synchronize()
    del a, b
    ha.close()
    hb.close()
    assert not mh._vmm_opened
    print(f"read_ok={ok}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
