"""eventfd hand-off between engine ranks and the layerwise worker over a UNIX
socket with SCM_RIGHTS (framing: 16-byte iiii header, per counter a 4-byte id
plus one descriptor batch, 1-byte ACK)."""
import os
import struct

from flexkv_b200.transfer.layerwise import EventfdReceiver, send_eventfds


def test_eventfds_cross_the_socket_and_stay_usable(tmp_path):
    installed = {}

    def install(counter, rank, layer, fd):
        installed[(counter, rank, layer)] = os.dup(fd)      # what the native group does

    path = str(tmp_path / "lw.sock")
    rx = EventfdReceiver(path, install)
    rx.start()
    try:
        L, C = 5, 3
        mine = {r: [[os.eventfd(0, os.EFD_NONBLOCK | os.EFD_SEMAPHORE) for _ in range(L)] for _ in range(C)]
                for r in range(2)}
        for r in range(2):
            send_eventfds(path, r, 2, mine[r])
        assert len(installed) == 2 * C * L and rx.ranks_seen == {0: C, 1: C}
        # a write on the worker's copy is seen on the engine's original descriptor
        os.write(installed[(1, 0, 3)], struct.pack("Q", 1))
        assert struct.unpack("Q", os.read(mine[0][1][3], 8))[0] == 1
        # nothing else fired
        for r in range(2):
            for c in range(C):
                for l in range(L):
                    try:
                        os.read(mine[r][c][l], 8)
                        assert False, "unexpected signal"
                    except BlockingIOError:
                        pass
    finally:
        rx.stop()
        for fd in installed.values():
            os.close(fd)


def test_socket_path_follows_the_reference_naming_rule(monkeypatch):
    from types import SimpleNamespace as NS
    from flexkv_b200.transfer.layerwise import build_layerwise_eventfd_socket_path as path
    monkeypatch.delenv("FLEXKV_LAYERWISE_SOCK", raising=False)
    monkeypatch.delenv("FLEXKV_LAYERWISE_EVENTFD_SOCKET", raising=False)
    one = NS(pp_size=1, dp_size=1, instance_num=1)
    assert path(0, 0, one) is None                               # same process: no socket
    monkeypatch.setenv("FLEXKV_LAYERWISE_SOCK", "/tmp/lw")
    assert path(3, 0, one) == "/tmp/lw.3"
    monkeypatch.setenv("FLEXKV_LAYERWISE_EVENTFD_SOCKET", "/run/fkv/eventfd.sock")
    assert path(0, 0, one) == "/run/fkv/eventfd.sock"
    assert path(2, 1, NS(pp_size=2, dp_size=4, instance_num=1)) == "/run/fkv/eventfd_pp1_dp2.sock"
    assert path(5, 0, NS(pp_size=1, dp_size=1, instance_num=2)) == "/run/fkv/eventfd_dp5.sock"
