"""Layerwise restore: the worker that executes LAYERWISE ops and the eventfd
hand-off with the engine process.

The engine's per-layer hook blocks on one eventfd per (counter, tp_rank, layer);
the worker signals each exactly once per restore, after that layer's KV has
landed on that rank's GPU (flexkv/transfer/layerwise.py:756-1059,
csrc/layerwise.cpp:105-137). The descriptors travel over a UNIX socket with
SCM_RIGHTS using the reference's framing (flexkv/transfer/layerwise.py:822-860):

    header  ``iiii``  = rank, tp_size, num_layers, num_counters   (16 bytes)
    then per counter: 4-byte counter id + one SCM_RIGHTS batch of num_layers fds
    reply   1 byte ACK
"""
from __future__ import annotations

import array
import os
import select
import socket
import struct
import threading
from typing import Callable, Dict, List, Optional, Sequence


from .. import _native
from ..common.config import GLOBAL_CONFIG_FROM_ENV
from ..common.debug import flexkv_logger
from ..common.transfer import LayerwiseTransferOp, TransferOp, WorkerKey
from .workers import OpOutcome, TransferWorker, _launch_cfg

HEADER = struct.Struct("iiii")
ACK = b"\x01"


def build_layerwise_eventfd_socket_path(dp_client_id: int, pp_rank: int, model_config) -> Optional[str]:
    """Where the layerwise worker of (dp client, pipeline stage) listens for the engine ranks' eventfds, or None
    when no socket is configured (worker and engine share a process). ``FLEXKV_LAYERWISE_EVENTFD_SOCKET`` follows
    the reference's naming rule: the given path, with ``_pp<rank>`` before the extension when there are several
    pipeline stages and ``_dp<id>`` when there are several data-parallel clients or instances
    (flexkv/transfer/layerwise.py:30-48). ``FLEXKV_LAYERWISE_SOCK`` is this package's older form,
    ``<path>.<dp client id>``."""
    base = os.environ.get("FLEXKV_LAYERWISE_EVENTFD_SOCKET", "")
    if base:
        suffix = ""
        if getattr(model_config, "pp_size", 1) > 1:
            suffix += f"_pp{pp_rank}"
        if getattr(model_config, "instance_num", 1) > 1 or getattr(model_config, "dp_size", 1) > 1:
            suffix += f"_dp{dp_client_id}"
        root, ext = os.path.splitext(base)
        return f"{root}{suffix}{ext}" if suffix else base
    sock = os.environ.get("FLEXKV_LAYERWISE_SOCK", "")
    return f"{sock}.{dp_client_id}" if sock else None


def send_eventfds(sock_path: str, rank: int, tp_size: int, fds_per_counter: Sequence[Sequence[int]],
                  timeout: float = 30.0) -> None:
    """Engine side: hands this rank's eventfds (``[counter][layer]``) to the worker."""
    num_counters = len(fds_per_counter)
    num_layers = len(fds_per_counter[0])
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
        s.settimeout(timeout)
        s.connect(sock_path)
        s.sendall(HEADER.pack(rank, tp_size, num_layers, num_counters))
        for c, fds in enumerate(fds_per_counter):
            if len(fds) != num_layers:
                raise ValueError("every counter needs one eventfd per layer")
            s.sendmsg([struct.pack("i", c)], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", fds))])
        if s.recv(1) != ACK:
            raise RuntimeError("layerwise worker did not acknowledge the eventfds")


def _recv_exact(conn: socket.socket, n: int) -> bytes:
    buf = b""
    while len(buf) < n:
        part = conn.recv(n - len(buf))
        if not part:
            raise ConnectionError("peer closed during the eventfd handshake")
        buf += part
    return buf


class EventfdReceiver:
    """Worker side: listens on a UNIX socket and installs received eventfds."""

    def __init__(self, sock_path: str, install: Callable[[int, int, int, int], None]) -> None:
        self.sock_path = sock_path
        self._install = install
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.ranks_seen: Dict[int, int] = {}
        if os.path.exists(sock_path):
            os.unlink(sock_path)
        self._srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._srv.bind(sock_path)
        self._srv.listen(64)

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, name="flexkv-eventfd-recv", daemon=True)
        self._thread.start()

    def _loop(self) -> None:
        while not self._stop.is_set():
            r, _, _ = select.select([self._srv], [], [], 0.2)
            if not r:
                continue
            conn, _ = self._srv.accept()
            try:
                self._handle(conn)
            except Exception as e:  # noqa: BLE001
                flexkv_logger.error("eventfd handshake failed: %s", e)
            finally:
                conn.close()

    def _handle(self, conn: socket.socket) -> None:
        conn.settimeout(30.0)
        rank, tp_size, num_layers, num_counters = HEADER.unpack(_recv_exact(conn, HEADER.size))
        for _ in range(num_counters):
            fds = array.array("i")
            msg, anc, _, _ = conn.recvmsg(4, socket.CMSG_LEN(num_layers * fds.itemsize))
            while len(msg) < 4:
                msg += _recv_exact(conn, 4 - len(msg))
            (counter,) = struct.unpack("i", msg)
            for level, ctype, data in anc:
                if level == socket.SOL_SOCKET and ctype == socket.SCM_RIGHTS:
                    fds.frombytes(data[:len(data) - (len(data) % fds.itemsize)])
            if len(fds) != num_layers:
                raise RuntimeError(f"expected {num_layers} eventfds for counter {counter}, got {len(fds)}")
            for layer, fd in enumerate(fds):
                self._install(counter, rank, layer, fd)     # the native side keeps a dup
                os.close(fd)
        self.ranks_seen[rank] = num_counters
        conn.sendall(ACK)

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        self._srv.close()
        try:
            os.unlink(self.sock_path)
        except OSError:
            pass


def build_layerwise_group(storage, model_config, key: WorkerKey, notify_mode: Optional[str] = None,
                          num_counters: int = 3, layers_per_batch: Optional[int] = None,
                          create_eventfds: bool = True):
    from ..common.storage import KVCacheLayoutType
    env = GLOBAL_CONFIG_FROM_ENV
    if layers_per_batch is None:
        # -1: one fused launch for small restores, one launch per layer for large ones
        layers_per_batch = int(os.environ.get("FLEXKV_LAYERWISE_LAYERS_PER_BATCH", -1))
    if storage.host.layout.is_multi_group:
        return _build_multi_group(storage, model_config, key, env, notify_mode, num_counters, create_eventfds)
    regs = storage.gpu_regs[key]
    ranks = sorted(regs)
    host, reg0 = storage.host, regs[ranks[0]]
    shared = model_config.use_mla or model_config.num_kv_heads == 1
    n_slices = 1 if shared else model_config.effective_tp_size
    if host.layout.type == KVCacheLayoutType.BLOCKFIRST:
        layer_stride, kv_stride, tp_stride = host.layer_stride // n_slices, host.kv_stride // n_slices, \
            host.block_bytes // n_slices
    else:
        layer_stride, kv_stride, tp_stride = host.layer_stride, host.kv_stride, host.chunk_bytes // n_slices
    host_d = dict(base=host.base, layer_stride=layer_stride, kv_stride=kv_stride, block_stride=host.block_bytes,
                  num_blocks=host.num_blocks)
    opts = dict(num_layers=reg0.num_layers, kv_dim=reg0.kv_dim, chunk_bytes=reg0.chunk_bytes,
                cpu_tp_stride=tp_stride, shared_kv=shared, h2d=_launch_cfg(env, True), d2h=_launch_cfg(env, False),
                max_blocks_per_op=max(4096, min(1 << 18, host.num_blocks)),
                notify_mode=notify_mode or env.layerwise_notify_mode, num_counters=num_counters,
                layers_per_batch=layers_per_batch, create_eventfds=create_eventfds)
    if "FLEXKV_LAYERWISE_FUSED_MAX_BYTES" in os.environ:
        # narrow grids (below 8 CTAs) restore with one launch per layer above this size; 64 MiB by default
        opts["fused_max_bytes"] = int(os.environ["FLEXKV_LAYERWISE_FUSED_MAX_BYTES"])
    if getattr(host, "quant", "none") == "bf16_xp":
        # packed host pool: the restore unpacks layer by layer and reads only the packed bytes
        from .compression import build_compressors
        spec = build_compressors(host, reg0.num_layers, reg0.kv_dim, len(ranks), shared).spec
        opts.update(size_table_ptr=host.size_table.data_ptr(), size_table_layers=spec.kernel_layers(),
                    size_table_rank_entries=spec.rank_offset_entries(1) if len(ranks) > 1 else 0,
                    codec_pipelines=int(os.environ.get("FLEXKV_QUANT_NUM_CTA", 64)))
    elif getattr(host, "quant", "none") != "none":
        raise ValueError(f"layerwise restore does not serve host pools in the {host.quant} format")
    return _native.C.LayerwiseGroup([regs[r].as_native() for r in ranks], host_d, opts)


def layer_members(model_config, groups) -> List[List[tuple]]:
    """``members[l]`` = the (group, layer inside the group) pairs that make up model layer ``l``.
    A group lists its model layers in ``LayerGroupSpec.layer_ids``; without the list its layers
    are model layers 0 .. n-1 (an indexer or a compressed copy beside every main-cache layer)
    (reference: csrc/layerwise.cpp:1313-1340)."""
    specs = model_config.layer_groups or []
    num_model_layers = int(model_config.num_layers)
    for g, spec in zip(groups, specs):
        ids = spec.layer_ids if spec.layer_ids is not None else range(g.num_layers)
        num_model_layers = max(num_model_layers, max(ids, default=-1) + 1)
    members: List[List[tuple]] = [[] for _ in range(num_model_layers)]
    for gid, g in enumerate(groups):
        spec = specs[gid] if gid < len(specs) else None
        ids = list(spec.layer_ids) if spec is not None and spec.layer_ids is not None else list(range(g.num_layers))
        if len(ids) != g.num_layers:
            raise ValueError(f"layer group {gid}: {len(ids)} layer ids for {g.num_layers} layers")
        for local, l in enumerate(ids):
            members[int(l)].append((gid, local))
    return members


def _build_multi_group(storage, model_config, key: WorkerKey, env, notify_mode, num_counters, create_eventfds):
    host = storage.host
    lay = host.layout
    per_rank = storage.gpu_group_regs.get(key, {})
    if not per_rank:
        raise ValueError("multi-group host pool but no per-group GPU registrations")
    ranks = sorted(per_rank)
    slice_bytes = host.block_bytes // lay.tp_slices
    shared = lay.tp_slices == 1
    groups = []
    for gid, g in enumerate(lay.groups):
        regs = []
        for r in ranks:
            reg = per_rank[r].get(gid)
            if reg is None:
                raise ValueError(f"rank {r} did not register layer group {gid}")
            regs.append(reg.as_native())
        groups.append(dict(
            gpus=regs,
            host=dict(base=host.base + g.offset_bytes, layer_stride=g.layer_stride_bytes, kv_stride=g.chunk_bytes,
                      block_stride=host.block_bytes, num_blocks=host.num_blocks),
            options=dict(num_layers=g.num_layers, kv_dim=g.kv_dim, chunk_bytes=g.chunk_bytes,
                         cpu_tp_stride=0 if shared else slice_bytes, shared_kv=shared)))
    members = layer_members(model_config, lay.groups)
    opts = dict(num_layers=len(members), kv_dim=1, chunk_bytes=16, h2d=_launch_cfg(env, True),
                d2h=_launch_cfg(env, False), max_blocks_per_op=max(4096, min(1 << 18, host.num_blocks)),
                notify_mode=notify_mode or env.layerwise_notify_mode, num_counters=num_counters,
                layers_per_batch=1, create_eventfds=create_eventfds)
    host_d = dict(base=host.base, layer_stride=host.block_bytes, kv_stride=0, block_stride=host.block_bytes,
                  num_blocks=host.num_blocks)
    return _native.C.LayerwiseGroup.multi_group(groups, [list(m) for m in members], host_d, opts)


class LayerwiseWorker(TransferWorker):
    """Executes LAYERWISE ops: SSD -> host for all layers, then host -> GPU per layer with signals."""

    name = "layerwise"

    def __init__(self, storage, model_config, key: WorkerKey, sock_path: Optional[str] = None, **kw) -> None:
        super().__init__()
        self.storage = storage
        self.group = build_layerwise_group(storage, model_config, key, **kw)
        self.receiver: Optional[EventfdReceiver] = None
        if sock_path:
            self.receiver = EventfdReceiver(sock_path, self.group.set_eventfd)
            self.receiver.start()
        self.last_result = None

    def execute(self, op: TransferOp) -> OpOutcome:
        assert isinstance(op, LayerwiseTransferOp)
        st = self.storage
        has_disk = op.src_block_ids_disk2h.size > 0
        if has_disk and st.ssd is None:
            return OpOutcome(False, error="layerwise op reads from SSD but no SSD tier is configured")
        r = self.group.restore(op.dst_block_ids_h2d, op.src_block_ids_h2d, op.counter_id,
                               st.ssd.engine if has_disk else None, st.ssd_layout_dict() if has_disk else None,
                               op.src_block_ids_disk2h if has_disk else None,
                               op.dst_block_ids_disk2h if has_disk else None)
        self.last_result = r
        nbytes = int(op.src_block_ids_h2d.size) * st.host.block_bytes
        return OpOutcome(r.status == 0, gpu_ms=r.total_ms, num_bytes=nbytes,
                         error="" if r.status == 0 else f"layerwise status 0x{r.status & 0xffffffff:x}")

    def update_gpu_ptrs(self, rank_index: int, ptrs, group_id: int = -1) -> None:
        if self.group.is_multi_group:
            self.group.update_group_gpu_ptrs(max(0, int(group_id)), rank_index, list(ptrs))
        else:
            self.group.update_gpu_ptrs(rank_index, list(ptrs))

    def close(self) -> None:
        if self.receiver is not None:
            self.receiver.stop()
