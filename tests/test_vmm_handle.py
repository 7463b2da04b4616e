"""Handles for memory from the CUDA virtual-memory API: the descriptor server (CPU), and on a GPU
an allocation made with cuMemCreate that a child process maps through the exported descriptor,
reads, rewrites and lets go (reference: tests/test_vmm_register.py, tests/test_memory_handle.py,
flexkv/common/memory_handle.py:466-545)."""
import os
import pickle
import subprocess
import sys

import pytest
import torch

from flexkv_b200.common import memory_handle as mh

HERE = os.path.dirname(os.path.abspath(__file__))


def test_descriptor_server_hands_out_duplicates_and_refuses_unknown_tokens(tmp_path, monkeypatch):
    monkeypatch.setenv("FLEXKV_VMM_FD_DIR", str(tmp_path))
    path = tmp_path / "payload"
    path.write_bytes(b"window into another process")
    fd = os.open(path, os.O_RDONLY)
    try:
        token, sock = mh.serve_fd(fd)
        assert sock == mh.fd_server_path(os.getpid()) and os.path.exists(sock)
        dup = mh.fetch_fd(sock, token)
        try:
            assert dup != fd and os.pread(dup, 64, 0) == b"window into another process"
        finally:
            os.close(dup)
        with pytest.raises(RuntimeError):
            mh.fetch_fd(sock, token + 12345)
        token2, sock2 = mh.serve_fd(fd)                      # same server, same token for the same descriptor
        assert (token2, sock2) == (token, sock)
    finally:
        mh.stop_fd_server()                                  # closes the served descriptors
    assert not os.path.exists(sock)
    with pytest.raises(OSError):
        os.fstat(fd)


def test_handle_pickles_with_its_vmm_fields():
    h = mh.TensorSharedHandle(mode="vmm_posix_fd", device_id=0, dtype=torch.bfloat16, shape=(4, 8), stride=(8, 1),
                              nbytes=64, pid=1, vmm_fd_token=7, vmm_fd_socket="/tmp/x.sock", vmm_base=1 << 30,
                              vmm_size=2 << 20, vmm_offset=4096)
    g = pickle.loads(pickle.dumps(h))
    assert g == h and g.dtype is torch.bfloat16 and g.vmm_offset == 4096


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [None, "vmm_posix_fd"])
def test_child_process_maps_a_cumemcreate_allocation(tmp_path, mode):
    C = mh._native.C
    va, size = C.vmm_alloc(3 << 20, 0, False)
    try:
        assert size >= 3 << 20 and C.vmm_is_vmm_pointer(va)
        plain = torch.zeros(16, device="cuda:0")
        assert not C.vmm_is_vmm_pointer(plain.data_ptr())    # cudaMalloc memory keeps the legacy IPC path
        whole = torch.as_tensor(mh.DeviceSpan(va, size), device="cuda:0")
        # two "layers" carved out of one allocation share one export
        a = whole[4096:4096 + (1 << 20)].view(torch.bfloat16).view(512, 1024)
        b = whole[2 << 20:(2 << 20) + 65536].view(torch.int32)
        a.copy_(torch.arange(512 * 1024, device="cuda:0").remainder(251).to(torch.bfloat16).view(512, 1024))
        b.fill_(7)
        torch.cuda.synchronize()
        ha, hb = mh.TensorSharedHandle.export(a, mode=mode), mh.TensorSharedHandle.export(b, mode=mode)
        assert ha.mode in ("vmm_posix_fd", "vmm_fabric") and ha.mode == hb.mode
        assert (ha.vmm_base, ha.vmm_offset, hb.vmm_offset) == (va, 4096, 2 << 20)
        if ha.mode == "vmm_posix_fd":
            assert ha.vmm_fd_token == hb.vmm_fd_token        # one descriptor per allocation
        assert ha.open() == a.data_ptr()                      # the exporter itself needs no mapping
        with open(tmp_path / "handles.pkl", "wb") as f:
            pickle.dump((ha, hb), f)
        out = subprocess.run([sys.executable, os.path.join(HERE, "mp_workers", "vmm_import_worker.py"),
                              str(tmp_path / "handles.pkl")], capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
        assert "read_ok=True" in out.stdout
        torch.cuda.synchronize()
        assert bool((b == 9).all())                           # the child's writes are visible here
        assert float(a[3, 5]) == -1.0
    finally:
        mh.stop_fd_server()
        mh._vmm_exports.clear()
        del whole, a, b
        torch.cuda.synchronize()
        C.vmm_free(va, size)
