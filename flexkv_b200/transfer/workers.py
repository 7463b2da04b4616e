"""Transfer workers: one thread per (worker key, direction) that executes ops
of one kind and reports an ``OpOutcome``.

Counterparts in the reference are worker *processes*
(flexkv/transfer/worker.py:709-1097 GPU<->host, :1099-1529 TP group,
:1531-1713 host<->SSD, :1948-2244 GDS, :1715-1946 remote file system).
A worker never drops an op: any exception becomes a failed outcome so that the
task layer can report FAILED instead of timing out
(flexkv/transfer/worker.py:612-619).
"""
from __future__ import annotations

import os
import queue
import threading
import time
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import numpy as np

from .. import _native
from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig
from ..common.debug import flexkv_logger
from ..common.storage import KVCacheLayoutType
from ..common.transfer import TransferOp, TransferType, WorkerKey


@dataclass
class OpOutcome:
    success: bool
    block_results: Optional[Tuple[bool, ...]] = None
    gpu_ms: float = 0.0
    num_bytes: int = 0
    error: str = ""


class TransferWorker:
    """Base: a FIFO of ops served by one thread."""

    name = "worker"

    def __init__(self) -> None:
        # SimpleQueue: put and get are C calls (no Python-level condition variable on the submit path)
        self._q: "queue.SimpleQueue[Optional[TransferOp]]" = queue.SimpleQueue()
        self._thread: Optional[threading.Thread] = None
        self._done_cb: Optional[Callable[[TransferOp, OpOutcome], None]] = None
        self.fail_next = 0          # host-side fault injection for tests: fail this many ops

    def start(self, done_cb: Callable[[TransferOp, OpOutcome], None]) -> None:
        self._done_cb = done_cb
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name=f"flexkv-{self.name}", daemon=True)
            self._thread.start()

    def stop(self) -> None:
        if self._thread is not None:
            self._q.put(None)
            self._thread.join(timeout=GLOBAL_CONFIG_FROM_ENV.worker_shutdown_timeout_s)
            self._thread = None
        self.close()

    def close(self) -> None:
        pass

    def submit(self, op: TransferOp) -> None:
        self._q.put(op)

    def _run(self) -> None:
        while True:
            op = self._q.get()
            if op is None:
                return
            try:
                if self.fail_next > 0:
                    self.fail_next -= 1
                    raise RuntimeError("injected worker failure")
                t0 = time.perf_counter()
                out = self.execute(op)
                if out.gpu_ms <= 0:            # IO workers have no device timing: report the time spent in the call
                    out.gpu_ms = (time.perf_counter() - t0) * 1e3
            except Exception as e:  # noqa: BLE001
                flexkv_logger.error("%s: op %d (%s) failed: %s", self.name, op.op_id, op.transfer_type.value, e)
                out = OpOutcome(False, error=str(e))
            self._done_cb(op, out)

    def execute(self, op: TransferOp) -> OpOutcome:
        raise NotImplementedError


# ------------------------------------------------------------------ GPU <-> host

_ENGINE_IDS = {"tma": 0, "simt": 1, "ce": 2, "auto": 3}


def _launch_cfg(env, h2d: bool) -> Dict[str, int]:
    """Engine per direction: FLEXKV_TRANSFER_ENGINE (tma | simt | ce | auto); the reference's
    FLEXKV_USE_CE_TRANSFER_H2D/D2H switches select the adaptive copy-engine router ("auto")
    for that direction (csrc/transfer.cu:164-313 chooses kernel vs copy engine the same way)."""
    engine = _ENGINE_IDS.get(env.transfer_engine, 0)
    if (env.use_ce_transfer_h2d if h2d else env.use_ce_transfer_d2h) and engine in (0, 1):
        engine = 3
    return dict(num_ctas=env.transfer_num_cta_h2d if h2d else env.transfer_num_cta_d2h,
                tile_bytes=env.transfer_tile_bytes, engine=engine)


def build_transfer_group(storage, model_config: ModelConfig, key: WorkerKey, high_priority: bool = False,
                         max_blocks_per_op: Optional[int] = None):
    """One native TransferGroup over every registered rank of ``key``."""
    env = GLOBAL_CONFIG_FROM_ENV
    regs = storage.gpu_regs[key]
    ranks = sorted(regs)
    host = storage.host
    reg0 = regs[ranks[0]]
    shared = model_config.use_mla or model_config.num_kv_heads == 1
    if host.layout.is_multi_group:
        raise ValueError("multi-group pools are served by MultiGroupGpuHostWorker")
    if host.quant != "none":
        raise ValueError("quantised pools are served by QuantGpuHostWorker")
    n_slices = 1 if shared else model_config.effective_tp_size
    if host.layout.type == KVCacheLayoutType.BLOCKFIRST:
        layer_stride, kv_stride = host.layer_stride // n_slices, host.kv_stride // n_slices
        tp_stride = host.block_bytes // n_slices
    else:
        layer_stride, kv_stride = host.layer_stride, host.kv_stride
        tp_stride = host.chunk_bytes // n_slices
    if not shared and host.chunk_bytes // n_slices != reg0.chunk_bytes:
        raise ValueError(f"host chunk {host.chunk_bytes} B / {n_slices} ranks does not match the GPU chunk "
                         f"{reg0.chunk_bytes} B")
    if shared and host.chunk_bytes != reg0.chunk_bytes:
        raise ValueError(f"host chunk {host.chunk_bytes} B does not match the GPU chunk {reg0.chunk_bytes} B")
    gpus = []
    for r in ranks:
        d = regs[r].as_native()
        gpus.append(d)
    host_d = dict(base=host.base + storage.pp_stage_offset(key.pp_rank), layer_stride=layer_stride,
                  kv_stride=kv_stride, block_stride=host.block_bytes, num_blocks=host.num_blocks)
    opts = dict(num_layers=reg0.num_layers, kv_dim=reg0.kv_dim, chunk_bytes=reg0.chunk_bytes,
                cpu_tp_stride=tp_stride, shared_kv=shared, shared_mode=env.kv_shared_across_ranks_mode,
                h2d=_launch_cfg(env, True), d2h=_launch_cfg(env, False), high_priority_stream=high_priority,
                **({"ce_max_copies": int(os.environ["FLEXKV_CE_SEGMENT_THRESHOLD"])}
                   if os.environ.get("FLEXKV_CE_SEGMENT_THRESHOLD") else {}),
                max_blocks_per_op=max_blocks_per_op or max(4096, min(1 << 18, host.num_blocks)))
    return _native.C.TransferGroup(gpus, host_d, opts)


class GpuHostWorker(TransferWorker):
    """H2D or D2H through the native transfer group (one kernel launch per GPU per op)."""

    def __init__(self, group, h2d: bool, block_bytes_per_rank: int, num_ranks: int) -> None:
        super().__init__()
        self.group = group
        self.h2d = h2d
        self.name = "h2d" if h2d else "d2h"
        self._bytes_per_block = block_bytes_per_rank * num_ranks

    def execute(self, op: TransferOp) -> OpOutcome:
        if self.h2d:
            cpu, gpu = op.src_block_ids, op.dst_block_ids
        else:
            gpu, cpu = op.src_block_ids, op.dst_block_ids
        if gpu.size != cpu.size:
            return OpOutcome(False, error=f"unbound GPU blocks: {gpu.size} vs {cpu.size}")
        nl = self.group_layers if op.num_layers < 0 else op.num_layers
        max_n = self.max_blocks
        status, ms = 0, 0.0
        tickets = []
        for lo in range(0, int(cpu.size), max_n):
            tickets.append(self.group.submit(gpu[lo:lo + max_n], cpu[lo:lo + max_n], self.h2d, op.layer_start, nl))
        for t in tickets:
            r = self.group.wait(t)
            status |= r.status if r.status >= 0 else (1 << 30)
            ms += r.gpu_ms
        ok = status == 0
        return OpOutcome(ok, gpu_ms=ms, num_bytes=int(cpu.size) * self._bytes_per_block,
                         error="" if ok else f"kernel status 0x{status:x}")

    group_layers = 0
    max_blocks = 1 << 16

    def update_gpu_ptrs(self, rank_index: int, ptrs) -> None:
        self.group.update_gpu_ptrs(rank_index, list(ptrs))


class HostEmulatedGpuWorker(TransferWorker):
    """GPU-less data plane: the registered "GPU" tensors are host tensors and
    the copy runs on CPU threads with the kernels' addressing. Serves CPU-only
    deployments of the control plane and the CPU test tier."""

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey, h2d: bool) -> None:
        super().__init__()
        self.h2d = h2d
        self.name = "h2d-host" if h2d else "d2h-host"
        self.regs = [storage.gpu_regs[key][r] for r in sorted(storage.gpu_regs[key])]
        host = storage.host
        self.host = host
        shared = model_config.use_mla or model_config.num_kv_heads == 1
        n_slices = 1 if shared else model_config.effective_tp_size
        if host.layout.type == KVCacheLayoutType.BLOCKFIRST:
            self.layer_stride, self.kv_stride = host.layer_stride // n_slices, host.kv_stride // n_slices
            self.tp_stride = host.block_bytes // n_slices
        else:
            self.layer_stride, self.kv_stride = host.layer_stride, host.kv_stride
            self.tp_stride = host.chunk_bytes // n_slices
        self.shared = shared
        self.pp_off = storage.pp_stage_offset(key.pp_rank)

    def execute(self, op: TransferOp) -> OpOutcome:
        if self.h2d:
            cpu, gpu = op.src_block_ids, op.dst_block_ids
        else:
            gpu, cpu = op.src_block_ids, op.dst_block_ids
        if gpu.size != cpu.size:
            return OpOutcome(False, error=f"unbound GPU blocks: {gpu.size} vs {cpu.size}")
        gpu = np.ascontiguousarray(gpu, dtype=np.int64)
        cpu = np.ascontiguousarray(cpu, dtype=np.int64)
        status, nbytes = 0, 0
        for i, reg in enumerate(self.regs):
            if self.shared and not self.h2d and i > 0:
                break       # identical KV on every rank: one writer is enough
            nl = reg.num_layers if op.num_layers < 0 else op.num_layers
            params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul,
                          idx_kv_mul=reg.idx_kv_mul, g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride,
                          g_block_stride=reg.block_stride, cpu_base=self.host.base, c_layer_stride=self.layer_stride,
                          c_kv_stride=self.kv_stride, c_block_stride=self.host.block_bytes,
                          c_off=self.pp_off + (0 if self.shared else i * self.tp_stride), gpu_blocks_ptr=gpu.ctypes.data,
                          cpu_blocks_ptr=cpu.ctypes.data, num_pairs=int(cpu.size), layer_start=op.layer_start,
                          num_layers=nl, kv_dim=reg.kv_dim, chunk_bytes=reg.chunk_bytes,
                          gpu_num_blocks=reg.num_blocks, cpu_num_blocks=self.host.num_blocks, h2d=int(self.h2d))
            status |= _native.C.host_kv_copy(params, 16)
            nbytes += int(cpu.size) * nl * reg.kv_dim * reg.chunk_bytes
        return OpOutcome(status == 0, num_bytes=nbytes, error="" if status == 0 else f"copy status 0x{status:x}")


class MultiGroupGpuHostWorker(TransferWorker):
    """H2D / D2H for caches made of several layer groups with different KV shapes (an indexer
    beside the main cache, compressed-KV groups storing fewer tokens per block). A host block is
    byte-flat: ``[rank slice][group][layer][kv][chunk]`` with per-group offsets; every group shares
    the op's block ids and is moved by its own launch per rank
    (reference format: flexkv/common/storage.py:87-127,249-286, flexkv/transfer/worker.py:886-921)."""

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey, h2d: bool) -> None:
        super().__init__()
        self.h2d = h2d
        self.name = "h2d-groups" if h2d else "d2h-groups"
        host = storage.host
        lay = host.layout
        per_rank = storage.gpu_group_regs.get(key, {})
        if not per_rank:
            raise ValueError("multi-group host pool but no per-group GPU registrations")
        self.ranks = sorted(per_rank)
        self.host = host
        self.slice_bytes = host.block_bytes // lay.tp_slices
        self.shared = lay.tp_slices == 1 and len(self.ranks) > 1
        self.groups = lay.groups
        self.regs = []                       # [rank index][group] -> registration
        for r in self.ranks:
            row = []
            for gid, g in enumerate(lay.groups):
                reg = per_rank[r].get(gid)
                if reg is None:
                    raise ValueError(f"rank {r} did not register layer group {gid}")
                if (reg.chunk_bytes, reg.num_layers, reg.kv_dim) != (g.chunk_bytes, g.num_layers, g.kv_dim):
                    raise ValueError(f"layer group {gid}: GPU tensors ({reg.num_layers} layers x {reg.kv_dim} x "
                                     f"{reg.chunk_bytes} B) do not match the host format ({g.num_layers} x "
                                     f"{g.kv_dim} x {g.chunk_bytes} B)")
                row.append(reg)
            self.regs.append(row)
        self.on_gpu = self.regs[0][0].device_id >= 0
        self.num_ctas = GLOBAL_CONFIG_FROM_ENV.transfer_num_cta_h2d if h2d else GLOBAL_CONFIG_FROM_ENV.transfer_num_cta_d2h
        self._streams, self._status = {}, {}
        if self.on_gpu:
            import torch
            self._torch = torch
            for row in self.regs:
                d = row[0].device_id
                self._streams[d] = torch.cuda.Stream(device=d)
                self._status[d] = torch.zeros(8, dtype=torch.int32, device=f"cuda:{d}")

    def execute(self, op: TransferOp) -> OpOutcome:
        cpu, gpu = (op.src_block_ids, op.dst_block_ids) if self.h2d else (op.dst_block_ids, op.src_block_ids)
        if gpu.size != cpu.size:
            return OpOutcome(False, error=f"unbound GPU blocks: {gpu.size} vs {cpu.size}")
        if self.on_gpu:
            g_ids = self._torch.from_numpy(np.ascontiguousarray(gpu, dtype=np.int64)).pin_memory()
            c_ids = self._torch.from_numpy(np.ascontiguousarray(cpu, dtype=np.int64)).pin_memory()
            g_ptr, c_ptr = g_ids.data_ptr(), c_ids.data_ptr()
        else:
            g_ids = np.ascontiguousarray(gpu, dtype=np.int64)
            c_ids = np.ascontiguousarray(cpu, dtype=np.int64)
            g_ptr, c_ptr = g_ids.ctypes.data, c_ids.ctypes.data
        status, nbytes, ms, evs = 0, 0, 0.0, []
        for i, row in enumerate(self.regs):
            if self.shared and not self.h2d and i > 0:
                break
            dev = row[0].device_id
            st = self._streams.get(dev)
            if self.on_gpu:
                e0, e1 = self._torch.cuda.Event(enable_timing=True), self._torch.cuda.Event(enable_timing=True)
                e0.record(st)
            for g, reg in zip(self.groups, row):
                params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul,
                              idx_kv_mul=reg.idx_kv_mul, g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride,
                              g_block_stride=reg.block_stride, cpu_base=self.host.base,
                              c_layer_stride=g.layer_stride_bytes, c_kv_stride=g.chunk_bytes,
                              c_block_stride=self.host.block_bytes,
                              c_off=g.offset_bytes + (0 if self.host.layout.tp_slices == 1
                                                      else self.ranks[i] * self.slice_bytes),
                              gpu_blocks_ptr=g_ptr, cpu_blocks_ptr=c_ptr, num_pairs=int(cpu.size), layer_start=0,
                              num_layers=g.num_layers, kv_dim=g.kv_dim, chunk_bytes=g.chunk_bytes,
                              gpu_num_blocks=reg.num_blocks, cpu_num_blocks=self.host.num_blocks, h2d=int(self.h2d))
                nbytes += int(cpu.size) * g.bytes
                if self.on_gpu:
                    params["status_ptr"] = self._status[dev].data_ptr()
                    with self._torch.cuda.device(dev):
                        _native.C.kv_copy(params, self.num_ctas, GLOBAL_CONFIG_FROM_ENV.transfer_tile_bytes, 0,
                                          st.cuda_stream)
                else:
                    status |= _native.C.host_kv_copy(params, 16)
            if self.on_gpu:
                e1.record(st)
                evs.append((e0, e1, dev))
        for e0, e1, dev in evs:
            e1.synchronize()
            ms = max(ms, e0.elapsed_time(e1))
            words = self._status[dev].tolist()
            status |= sum(1 << b for b, w in enumerate(words) if w)
            if status:
                self._status[dev].zero_()
        return OpOutcome(status == 0, gpu_ms=ms, num_bytes=nbytes,
                         error="" if status == 0 else f"copy status 0x{status:x}")


class QuantGpuHostWorker(TransferWorker):
    """H2D / D2H for host pools kept in a packed form: block-scaled fp8 (lossy) or
    the lossless exponent-packing codec. The copy kernel packs on the way out and
    unpacks on the way in, one launch per rank and op
    (reference strategy plug-in point: flexkv/transfer/compression/common/strategy.py:13-51)."""

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey, h2d: bool) -> None:
        super().__init__()
        import torch
        self.h2d = h2d
        self.name = ("h2d-" if h2d else "d2h-") + storage.host.quant
        self.regs = [storage.gpu_regs[key][r] for r in sorted(storage.gpu_regs[key])]
        host = storage.host
        if host.layout.type != KVCacheLayoutType.BLOCKFIRST:
            raise ValueError("packed host pools use the BLOCKFIRST host layout")
        self.codec = host.quant
        self.layers_total = self.regs[0].num_layers
        self.shared = model_config.use_mla or model_config.num_kv_heads == 1
        from .compression import build_compressors
        self.strategy = build_compressors(host, self.layers_total, self.regs[0].kv_dim, len(self.regs), self.shared)
        self.strategy.attach(self)
        n = 1 if self.shared else model_config.effective_tp_size
        self.host = host
        self.layer_stride, self.kv_stride, self.tp_stride = host.layer_stride // n, host.kv_stride // n, \
            host.block_bytes // n
        # Tile pipelines per launch (two share an SM in the lossless codec's kernel). Measured on B200 with
        # Llama-3-8B blocks: 80 pipelines (40 SMs) put both directions on the link's plateau for SM-issued
        # traffic; the fp8 kernel needs fewer (its CTAs are single pipelines)
        dflt = 80 if storage.host.quant == "bf16_xp" else (32 if h2d else 48)
        self.num_ctas = int(os.environ.get("FLEXKV_QUANT_NUM_CTA", dflt))
        self._torch = torch
        self.streams = {r.device_id: torch.cuda.Stream(device=r.device_id) for r in self.regs}
        self.status = {r.device_id: torch.zeros(8, dtype=torch.int32, device=f"cuda:{r.device_id}") for r in self.regs}

    def execute(self, op: TransferOp) -> OpOutcome:
        torch = self._torch
        if self.h2d:
            cpu, gpu = op.src_block_ids, op.dst_block_ids
        else:
            gpu, cpu = op.src_block_ids, op.dst_block_ids
        if gpu.size != cpu.size:
            return OpOutcome(False, error=f"unbound GPU blocks: {gpu.size} vs {cpu.size}")
        keep, evs, nbytes = [], [], 0
        g_ids = torch.from_numpy(np.ascontiguousarray(gpu, dtype=np.int64)).pin_memory()
        c_ids = torch.from_numpy(np.ascontiguousarray(cpu, dtype=np.int64)).pin_memory()
        for i, reg in enumerate(self.regs):
            if self.shared and not self.h2d and i > 0:
                break
            nl = reg.num_layers if op.num_layers < 0 else op.num_layers
            params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul,
                          idx_kv_mul=reg.idx_kv_mul, g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride,
                          g_block_stride=reg.block_stride, cpu_base=self.host.base, c_layer_stride=self.layer_stride,
                          c_kv_stride=self.kv_stride, c_block_stride=self.host.block_bytes,
                          c_off=0 if self.shared else i * self.tp_stride, gpu_blocks_ptr=g_ids.data_ptr(),
                          cpu_blocks_ptr=c_ids.data_ptr(), num_pairs=int(cpu.size), layer_start=op.layer_start,
                          num_layers=nl, kv_dim=reg.kv_dim, chunk_bytes=reg.chunk_bytes,
                          gpu_num_blocks=reg.num_blocks, cpu_num_blocks=self.host.num_blocks,
                          status_ptr=self.status[reg.device_id].data_ptr(), h2d=int(self.h2d))
            st = self.streams[reg.device_id]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(reg.device_id):
                e0.record(st)
                self.strategy.run(params, i, self.num_ctas, st.cuda_stream)
                e1.record(st)
            evs.append((e0, e1, reg.device_id))
            nbytes += int(cpu.size) * nl * reg.kv_dim * reg.chunk_bytes
        status, ms = 0, 0.0
        for e0, e1, dev in evs:
            e1.synchronize()
            ms = max(ms, e0.elapsed_time(e1))
            words = self.status[dev].tolist()
            status |= sum(1 << b for b, w in enumerate(words) if w)
            if status:
                self.status[dev].zero_()
        return OpOutcome(status == 0, gpu_ms=ms, num_bytes=nbytes,
                         error="" if status == 0 else f"quant kernel status 0x{status:x}")


class NvlsFanoutWorker(TransferWorker):
    """H2D for a shared-KV tensor-parallel group whose caches are symmetric memory: the issuing rank's kernel
    reads each host block over PCIe once and `multimem.st` replicates it into every rank's cache through
    NVSwitch, then raises the ranks' completion flag to the op's epoch (``last_epoch``). The reference reads the
    same host bytes once per rank (csrc/layerwise.cpp:1142-1165, csrc/tp_transfer_thread_group.cpp:221-323).
    The op completes after the issuing GPU has finished the launch; ranks in other processes may also wait on
    the flag (``parallel.nvls.wait_flag``)."""

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey) -> None:
        super().__init__()
        import torch
        self._torch = torch
        self.name = "h2d-nvls-fanout"
        regs = storage.gpu_regs[key]
        self.reg = regs[sorted(regs)[0]]
        if len(self.reg.mc_ptrs) != len(self.reg.ptrs) or not self.reg.mc_flag_ptr:
            raise ValueError("multicast registration needs one multicast address per tensor and a flag address")
        host = storage.host
        layer_stride, kv_stride = host.layer_stride, host.kv_stride     # shared KV: every rank reads whole chunks
        if host.chunk_bytes != self.reg.chunk_bytes:
            raise ValueError(f"host chunk {host.chunk_bytes} B does not match the GPU chunk {self.reg.chunk_bytes} B")
        self.host = dict(base=host.base + storage.pp_stage_offset(key.pp_rank), layer_stride=layer_stride,
                         kv_stride=kv_stride, block_stride=host.block_bytes, num_blocks=host.num_blocks)
        env = GLOBAL_CONFIG_FROM_ENV
        self.num_ctas = env.transfer_num_cta_h2d
        self.tile_bytes = env.transfer_tile_bytes
        dev = self.reg.device_id
        self.stream = torch.cuda.Stream(device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=f"cuda:{dev}")
        self.scratch = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        self.last_epoch = 0
        self.num_ranks = model_config.effective_tp_size_per_node

    def execute(self, op: TransferOp) -> OpOutcome:
        torch = self._torch
        cpu, gpu = op.src_block_ids, op.dst_block_ids
        if gpu.size != cpu.size:
            return OpOutcome(False, error=f"unbound GPU blocks: {gpu.size} vs {cpu.size}")
        reg, h = self.reg, self.host
        g_ids = torch.from_numpy(np.ascontiguousarray(gpu, dtype=np.int64)).pin_memory()
        c_ids = torch.from_numpy(np.ascontiguousarray(cpu, dtype=np.int64)).pin_memory()
        nl = reg.num_layers - op.layer_start if op.num_layers < 0 else op.num_layers
        self.last_epoch += 1
        params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], mc_ptrs=[int(p) for p in reg.mc_ptrs],
                      idx_layer_mul=reg.idx_layer_mul, idx_kv_mul=reg.idx_kv_mul, g_layer_stride=reg.layer_stride,
                      g_kv_stride=reg.kv_stride, g_block_stride=reg.block_stride, cpu_base=h["base"],
                      c_layer_stride=h["layer_stride"], c_kv_stride=h["kv_stride"], c_block_stride=h["block_stride"],
                      c_off=0, gpu_blocks_ptr=g_ids.data_ptr(), cpu_blocks_ptr=c_ids.data_ptr(),
                      num_pairs=int(cpu.size), layer_start=op.layer_start, num_layers=nl, kv_dim=reg.kv_dim,
                      chunk_bytes=reg.chunk_bytes, gpu_num_blocks=reg.num_blocks, cpu_num_blocks=h["num_blocks"],
                      status_ptr=self.status.data_ptr(), h2d=1, done_counter_ptr=self.scratch.data_ptr(),
                      epoch=self.last_epoch)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.device(reg.device_id):
            e0.record(self.stream)
            _native.C.kv_fanout(params, 0, int(reg.mc_flag_ptr), self.num_ctas, self.tile_bytes,
                                self.stream.cuda_stream)
            e1.record(self.stream)
        e1.synchronize()
        words = self.status.tolist()
        status = sum(1 << b for b, w in enumerate(words) if w)
        if status:
            self.status.zero_()
        nbytes = int(cpu.size) * nl * reg.kv_dim * reg.chunk_bytes
        return OpOutcome(status == 0, gpu_ms=e0.elapsed_time(e1), num_bytes=nbytes * self.num_ranks,
                         error="" if status == 0 else f"fan-out kernel status 0x{status:x}")


# ------------------------------------------------------------------ GPU <-> GPU (NVLink)

def even_tile_bytes(chunk_bytes: int, limit: int = 24576, fallback: int = 16384) -> int:
    """Largest tile of at most ``limit`` bytes that cuts a chunk into equal 16-byte-aligned pieces (no ragged last
    tile): 73,728-byte MLA chunks -> 24,576, 32 KiB chunks -> 16,384."""
    for n in range(1, 65):
        if chunk_bytes % n == 0:
            t = chunk_bytes // n
            if t <= limit and t % 16 == 0 and t >= 1024:
                return t
    return fallback


class PeerD2DWorker(TransferWorker):
    """Pulls blocks out of other ranks' paged caches over NVLink peer memory
    (one launch per owner rank; source and destination layouts are independent)."""

    name = "peer-d2d"

    def __init__(self, storage, model_config: ModelConfig, tp_rank: int = 0) -> None:
        super().__init__()
        env = GLOBAL_CONFIG_FROM_ENV
        keys = sorted(k for k in storage.gpu_regs if tp_rank in storage.gpu_regs[k])
        self.rank_of = {k.dp_client_id: i for i, k in enumerate(keys)}
        regs = [storage.gpu_regs[k][tp_rank] for k in keys]
        r0 = regs[0]
        for r in regs:
            if (r.chunk_bytes, r.num_layers, r.kv_dim) != (r0.chunk_bytes, r0.num_layers, r0.kv_dim):
                raise ValueError("peer ranks must share the KV chunk geometry")
        self.num_layers = r0.num_layers
        self.bytes_per_block = r0.num_layers * r0.kv_dim * r0.chunk_bytes
        # NVLink needs more loads in flight than PCIe: measured on two B200 with 72 KiB MLA chunks, 64 single-warp
        # CTAs with 16 KiB tiles reach 548 GB/s, 128 CTAs with tiles that divide the chunk evenly 772 GB/s, the
        # rate of one contiguous peer copy (770 GB/s)
        tile = int(os.environ.get("FLEXKV_PEER_TILE_BYTES", 0)) or even_tile_bytes(r0.chunk_bytes)
        self.copier = _native.C.PeerCopier([r.as_native() for r in regs], r0.num_layers, r0.kv_dim, r0.chunk_bytes,
                                           num_ctas=int(os.environ.get("FLEXKV_PEER_NUM_CTA", 128)),
                                           tile_bytes=tile, engine=0,
                                           max_blocks_per_op=max(4096, max(r.num_blocks for r in regs)))

    def update_gpu_ptrs_for(self, dp_client_id: int, ptrs) -> None:
        self.copier.update_gpu_ptrs(self.rank_of[dp_client_id], list(ptrs))

    def execute(self, op: TransferOp) -> OpOutcome:
        src, dst, owners = op.src_block_ids, op.dst_block_ids, op.remote_node_ids
        if dst.size != src.size or owners is None or owners.size != src.size:
            return OpOutcome(False, error="peer op needs bound destination blocks and one owner per block")
        me = self.rank_of[op.dp_client_id]
        status, ms = 0, 0.0
        nl = self.num_layers if op.num_layers < 0 else op.num_layers
        for owner in np.unique(owners):
            sel = owners == owner
            r = self.copier.pull(me, self.rank_of[int(owner)], np.ascontiguousarray(dst[sel]),
                                 np.ascontiguousarray(src[sel]), op.layer_start, nl)
            status |= r.status if r.status >= 0 else (1 << 30)
            ms += r.gpu_ms
        return OpOutcome(status == 0, gpu_ms=ms, num_bytes=int(src.size) * self.bytes_per_block,
                         error="" if status == 0 else f"peer copy status 0x{status:x}")


# ------------------------------------------------------------------ host <-> SSD

class SsdWorker(TransferWorker):
    def __init__(self, storage, is_read: bool) -> None:
        super().__init__()
        self.storage = storage
        self.is_read = is_read
        self.name = "disk2h" if is_read else "h2disk"

    def _move_size_tables(self, cpu: np.ndarray, ssd: np.ndarray, ok: np.ndarray) -> None:
        """Packed pools: a block's tile sizes travel with it between the host and SSD tables
        (flexkv/transfer/compression/ans/ans_utils.py:215-218)."""
        st = self.storage
        if st.ssd_size_table is None:
            return
        good = ok.astype(bool)
        ht = st.host.size_table.view(st.host.num_blocks, -1).numpy()
        if self.is_read:
            ht[cpu[good]] = st.ssd_size_table[ssd[good]]
        else:
            st.ssd_size_table[ssd[good]] = ht[cpu[good]]

    def execute(self, op: TransferOp) -> OpOutcome:
        st = self.storage
        if self.is_read:
            ssd, cpu = op.src_block_ids, op.dst_block_ids
        else:
            cpu, ssd = op.src_block_ids, op.dst_block_ids
        lay = st.ssd_layout_dict()
        nl = lay["num_layers"] if op.num_layers < 0 else op.num_layers
        geo = st.packed_ssd_geometry() if (op.layer_start == 0 and nl == lay["num_layers"]) else None
        if geo is not None:
            # packed pool: only the used bytes of every tile cross the SSD interface, one run per block
            cpu = np.ascontiguousarray(cpu, dtype=np.int64)
            ssd = np.ascontiguousarray(ssd, dtype=np.int64)
            if self.is_read:
                rows = st.ssd_size_table[ssd]
            else:
                rows = st.host.size_table.view(st.host.num_blocks, -1).numpy()[cpu]
            before = st.ssd.engine.bytes_read if self.is_read else st.ssd.engine.bytes_written
            nfail, ok = st.ssd.engine.transfer_packed(st.host.base, cpu, ssd, self.is_read, geo, rows)
            self._move_size_tables(cpu, ssd, ok)
            after = st.ssd.engine.bytes_read if self.is_read else st.ssd.engine.bytes_written
            return OpOutcome(nfail == 0, block_results=tuple(bool(x) for x in ok), num_bytes=int(after - before),
                             error="" if nfail == 0 else f"{nfail} block(s) failed")
        nfail, ok = st.ssd.engine.transfer(st.host.base, cpu, ssd, self.is_read, lay, op.layer_start, nl)
        self._move_size_tables(cpu, ssd, ok)
        return OpOutcome(nfail == 0, block_results=tuple(bool(x) for x in ok),
                         num_bytes=int((len(ok) - nfail)) * st.ssd.block_bytes,
                         error="" if nfail == 0 else f"{nfail} block(s) failed")


class RemoteWorker(TransferWorker):
    """H2REMOTE / REMOTE2H through a remote back end (shared files or a key-addressed
    store). Reports a per-block result list; any failed block fails the op
    (flexkv/transfer/worker.py:1715-1946,3875-4092)."""

    def __init__(self, storage, backend, to_host: bool, registry=None) -> None:
        super().__init__()
        self.storage, self.backend, self.to_host = storage, backend, to_host
        self.name = "remote2h" if to_host else "h2remote"
        self.registry = registry
        self._peer_files: Dict[int, Any] = {}

    def _files_of(self, nid: int):
        """The files node `nid` wrote to the shared remote file system, opened read-only once."""
        ent = self._peer_files.get(nid)
        if ent is not None:
            return ent
        import json
        from ..external.remote_store import PeerRemoteFiles
        meta = self.registry.get_node_meta(nid) if self.registry is not None else None
        if not meta or not meta.get("remote_files"):
            raise RuntimeError(f"node {nid} has no remote files in the registry")
        if int(meta["remote_block_bytes"]) != self.storage.host.block_bytes or \
                meta.get("codec", "none") != self.storage.host.quant:
            raise RuntimeError(f"node {nid} uses a different block format")
        ent = PeerRemoteFiles(json.loads(meta["remote_files"]), int(meta["remote_block_bytes"]),
                              int(meta["remote_num_blocks"]))
        self._peer_files[nid] = ent
        return ent

    def _execute_peer(self, op: TransferOp) -> OpOutcome:
        """REMOTE2H whose blocks live in other nodes' files (``remote_node_ids`` names the owner per block)."""
        host = self.storage.host
        src = np.asarray(op.src_block_ids, dtype=np.int64)
        dst = np.asarray(op.dst_block_ids, dtype=np.int64)
        owners = np.asarray(op.remote_node_ids, dtype=np.int64)
        n = len(src)
        if len(owners) != n or len(dst) != n:
            return OpOutcome(False, error="peer remote op without owner ids")
        results, err = [False] * n, ""
        for nid in np.unique(owners).tolist():
            sel = np.nonzero(owners == nid)[0]
            try:
                files = self._files_of(int(nid))
                got = files.get(src[sel].tolist(), [host.block_view(int(b)) for b in dst[sel]])
                for k, good in zip(sel.tolist(), got):
                    results[k] = bool(good)
            except (RuntimeError, OSError, ValueError) as e:
                err = str(e)
                self._peer_files.pop(int(nid), None)
        ok = all(results)
        if not ok and op.allow_partial and results and results[0]:
            return OpOutcome(True, block_results=tuple(results), num_bytes=sum(results) * host.block_bytes)
        return OpOutcome(ok, block_results=tuple(results), num_bytes=sum(results) * host.block_bytes,
                         error="" if ok else f"{n - sum(results)} block(s) of other nodes' remote files failed: {err}")

    def close(self) -> None:
        for f in self._peer_files.values():
            f.close()
        self._peer_files.clear()

    def execute(self, op: TransferOp) -> OpOutcome:
        if self.to_host and op.remote_node_ids is not None:
            return self._execute_peer(op)
        host = self.storage.host
        if self.to_host:
            rids, cpu = op.src_block_ids, op.dst_block_ids
        else:
            cpu, rids = op.src_block_ids, op.dst_block_ids
        ids = op.block_hashes if self.backend.key_addressed else rids
        if ids is None or len(ids) != len(cpu):
            return OpOutcome(False, error="remote op without matching ids")
        views = [host.block_view(int(b)) for b in cpu]
        res = self.backend.get(list(ids), views) if self.to_host else self.backend.put(list(ids), views)
        ok = all(res)
        if not ok and op.allow_partial and self.to_host and res and res[0]:
            # the planner keeps the longest successful prefix (prefetch); the op itself counts as done
            return OpOutcome(True, block_results=tuple(bool(r) for r in res), num_bytes=sum(res) * host.block_bytes)
        return OpOutcome(ok, block_results=tuple(bool(r) for r in res), num_bytes=sum(res) * host.block_bytes,
                         error="" if ok else f"{len(res) - sum(res)} remote block(s) failed")


class SwaWorker(TransferWorker):
    """Moves sliding-window pages between the GPU window pool and the host window pool
    (ops flagged ``is_swa``; ids are window page ids on the GPU side and slot ids on the
    host side). Pages are small and few, so one plain copy-kernel launch per rank and op
    on its own stream is enough; host-resident stand-ins go through the CPU oracle."""

    name = "swa"

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey) -> None:
        super().__init__()
        self.storage = storage
        self.regs = [storage.swa_regs[key][r] for r in sorted(storage.swa_regs[key])]
        # every group of a rank's slot (window KV first, then sidecar state) moves with its own launch
        self.group_regs = [[storage.swa_group_regs[key][r][g] for g in sorted(storage.swa_group_regs[key][r])]
                           for r in sorted(storage.swa_regs[key])]
        self.shared = model_config.use_mla or model_config.num_kv_heads == 1
        self.on_gpu = self.regs[0].device_id >= 0
        self._streams, self._status = {}, {}
        if self.on_gpu:
            import torch
            self._torch = torch
            for r in self.regs:
                self._streams[r.device_id] = torch.cuda.Stream(device=r.device_id)
                self._status[r.device_id] = torch.zeros(8, dtype=torch.int32, device=f"cuda:{r.device_id}")

    def execute(self, op: TransferOp) -> OpOutcome:
        h2d = op.transfer_type == TransferType.H2D
        if op.transfer_type in (TransferType.H2DISK, TransferType.DISK2H):
            return self._disk(op)
        if op.transfer_type in (TransferType.H2REMOTE, TransferType.REMOTE2H):
            return self._remote(op)
        if op.transfer_type not in (TransferType.H2D, TransferType.D2H):
            return OpOutcome(False, error=f"window ops on {op.transfer_type.value} are not built")
        slots, pages = (op.src_block_ids, op.dst_block_ids) if h2d else (op.dst_block_ids, op.src_block_ids)
        if slots.size != pages.size or slots.size == 0:
            return OpOutcome(False, error=f"unbound window pages: {pages.size} vs {slots.size} slots")
        pool = self.storage.swa_host
        nbytes, status, ms = 0, 0, 0.0
        if self.on_gpu:
            g_ids = self._torch.from_numpy(np.ascontiguousarray(pages, dtype=np.int64)).pin_memory()
            c_ids = self._torch.from_numpy(np.ascontiguousarray(slots, dtype=np.int64)).pin_memory()
            g_ptr, c_ptr = g_ids.data_ptr(), c_ids.data_ptr()
        else:
            g_ids = np.ascontiguousarray(pages, dtype=np.int64)
            c_ids = np.ascontiguousarray(slots, dtype=np.int64)
            g_ptr, c_ptr = g_ids.ctypes.data, c_ids.ctypes.data
        evs = []
        for i, groups in enumerate(self.group_regs):
            if self.shared and not h2d and i > 0:
                break
            dev_id = groups[0].device_id
            if self.on_gpu:
                st = self._streams[dev_id]
                e0, e1 = self._torch.cuda.Event(enable_timing=True), self._torch.cuda.Event(enable_timing=True)
                e0.record(st)
            for reg in groups:
                g = max(0, int(reg.group_id))
                params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul,
                              idx_kv_mul=reg.idx_kv_mul, g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride,
                              g_block_stride=reg.block_stride, cpu_base=pool.base,
                              c_layer_stride=pool.group_page_bytes[g], c_kv_stride=0, c_block_stride=pool.slot_bytes,
                              c_off=(0 if self.shared else i * pool.rank_slot_bytes) + pool.group_offsets[g],
                              gpu_blocks_ptr=g_ptr, cpu_blocks_ptr=c_ptr, num_pairs=int(slots.size), layer_start=0,
                              num_layers=reg.num_layers, kv_dim=1, chunk_bytes=reg.chunk_bytes,
                              gpu_num_blocks=reg.num_blocks, cpu_num_blocks=pool.num_slots, h2d=int(h2d))
                nbytes += int(slots.size) * reg.num_layers * reg.chunk_bytes
                if not self.on_gpu:
                    status |= _native.C.host_kv_copy(params, 16)
                    continue
                params["status_ptr"] = self._status[dev_id].data_ptr()
                with self._torch.cuda.device(dev_id):
                    _native.C.kv_copy(params, 4, 16384, 0, st.cuda_stream)
            if self.on_gpu:
                e1.record(st)
                evs.append((e0, e1, dev_id))
        for e0, e1, dev in evs:
            e1.synchronize()
            ms = max(ms, e0.elapsed_time(e1))
            words = self._status[dev].tolist()
            status |= sum(1 << b for b, w in enumerate(words) if w)
            if status:
                self._status[dev].zero_()
        return OpOutcome(status == 0, gpu_ms=ms, num_bytes=nbytes,
                         error="" if status == 0 else f"window copy status 0x{status:x}")


    def _disk(self, op: TransferOp) -> OpOutcome:
        """Host window slots <-> slots of the SSD window file (whole slots, the SSD tier's IO engine)."""
        st = self.storage
        if st.swa_ssd is None or st.swa_host is None:
            return OpOutcome(False, error="window op on the SSD tier but no SSD window pool is configured")
        read = op.transfer_type == TransferType.DISK2H
        host, disk = (op.dst_block_ids, op.src_block_ids) if read else (op.src_block_ids, op.dst_block_ids)
        if host.size != disk.size or host.size == 0:
            return OpOutcome(False, error=f"window disk op with {host.size} host and {disk.size} SSD slots")
        nfail, ok = st.swa_ssd.engine.transfer(st.swa_host.base, np.ascontiguousarray(host, dtype=np.int64),
                                               np.ascontiguousarray(disk, dtype=np.int64), read,
                                               st.swa_ssd_layout_dict(), 0, 1)
        return OpOutcome(nfail == 0, num_bytes=int(len(ok) - nfail) * st.swa_ssd.block_bytes,
                         error="" if nfail == 0 else f"{nfail} window slot(s) failed")


    def _remote(self, op: TransferOp) -> OpOutcome:
        """Host window slots <-> slots of the window file on the remote mount (positional reads and writes)."""
        import ctypes
        st = self.storage
        if not st.swa_remote_path or st.swa_host is None:
            return OpOutcome(False, error="window op on the remote tier but no remote window file is configured")
        read = op.transfer_type == TransferType.REMOTE2H
        host, far = (op.dst_block_ids, op.src_block_ids) if read else (op.src_block_ids, op.dst_block_ids)
        if host.size != far.size or host.size == 0:
            return OpOutcome(False, error=f"window remote op with {host.size} host and {far.size} remote slots")
        b = st.swa_host.slot_bytes
        bad = 0
        fd = os.open(st.swa_remote_path, os.O_RDWR)
        try:
            for h, r in zip(host.tolist(), far.tolist()):
                if not (0 <= h < st.swa_host.num_slots and 0 <= r < st.swa_remote_slots):
                    bad += 1
                    continue
                view = (ctypes.c_char * b).from_address(st.swa_host.base + h * b)
                try:
                    if read:
                        data = os.pread(fd, b, r * b)
                        if len(data) != b:
                            bad += 1
                            continue
                        ctypes.memmove(view, data, b)
                    elif os.pwrite(fd, bytes(view), r * b) != b:
                        bad += 1
                except OSError:
                    bad += 1
        finally:
            os.close(fd)
        return OpOutcome(bad == 0, num_bytes=(int(host.size) - bad) * b,
                         error="" if bad == 0 else f"{bad} window slot(s) failed")


class PeerHostWorker(TransferWorker):
    """PEERH2H: pulls blocks out of other nodes' host pools into this node's pool.
    Inside one box every pool is a shared-memory file whose name the owner published in
    the registry; blocks are grouped by owner and contiguous segment and copied with
    plain memcpy (the reference moves them with RDMA reads, flexkv/transfer/worker.py:
    2920-3029, segment grouping flexkv/transfer/utils.py:41-98). The owner's lease keeps
    the blocks in place while they are read."""

    name = "peerh2h"

    def __init__(self, storage, registry) -> None:
        super().__init__()
        self.storage, self.registry = storage, registry
        self._maps: Dict[int, Tuple[np.ndarray, int, int]] = {}

    def _pool_of(self, nid: int):
        ent = self._maps.get(nid)
        if ent is not None:
            return ent
        meta = self.registry.get_node_meta(nid)
        if not meta or not meta.get("pool_file"):
            raise RuntimeError(f"node {nid} has no host pool in the registry")
        if int(meta["block_bytes"]) != self.storage.host.block_bytes or \
                meta.get("codec", "none") != self.storage.host.quant:
            raise RuntimeError(f"node {nid} uses a different host block format")
        mm = np.memmap(meta["pool_file"], dtype=np.uint8, mode="r",
                       shape=(int(meta["num_blocks"]) * int(meta["block_bytes"]),))
        ent = (mm, int(meta["block_bytes"]), int(meta["num_blocks"]))
        self._maps[nid] = ent
        return ent

    def execute(self, op: TransferOp) -> OpOutcome:
        src, dst, nids = op.src_block_ids, op.dst_block_ids, op.remote_node_ids
        if nids is None or len(nids) != len(src) or len(src) != len(dst):
            return OpOutcome(False, error="peer host op without owner ids")
        host = self.storage.host
        bb = host.block_bytes
        n = len(src)
        results = [False] * n
        err = ""
        src = np.asarray(src, dtype=np.int64)
        dst = np.asarray(dst, dtype=np.int64)
        owners = np.asarray(nids, dtype=np.int64)
        for nid in np.unique(owners).tolist():
            sel = np.nonzero(owners == nid)[0]
            try:
                pool, _, nblk = self._pool_of(int(nid))
                s_ids = np.ascontiguousarray(src[sel])
                d_ids = np.ascontiguousarray(dst[sel])
                if s_ids.min() < 0 or s_ids.max() >= nblk:
                    raise RuntimeError(f"block {int(s_ids.max())} outside node {nid}'s pool")
                if d_ids.min() < 0 or d_ids.max() >= host.num_blocks:
                    raise RuntimeError(f"destination block {int(d_ids.max())} outside the host pool")
                # the owner's pool plays the paged side of the host copy helper (one tensor, whole blocks as
                # chunks), so the blocks move on the helper's thread pool instead of one memcpy at a time
                params = dict(gpu_ptrs=[int(pool.ctypes.data)], idx_layer_mul=0, idx_kv_mul=0, g_layer_stride=0,
                              g_kv_stride=0, g_block_stride=bb, cpu_base=host.base, c_layer_stride=0, c_kv_stride=0,
                              c_block_stride=bb, c_off=0, gpu_blocks_ptr=s_ids.ctypes.data,
                              cpu_blocks_ptr=d_ids.ctypes.data, num_pairs=int(sel.size), layer_start=0, num_layers=1,
                              kv_dim=1, chunk_bytes=bb, gpu_num_blocks=nblk, cpu_num_blocks=host.num_blocks, h2d=0)
                status = _native.C.host_kv_copy(params, 16)
                if status != 0:
                    raise RuntimeError(f"host copy status 0x{status:x}")
                for k in sel.tolist():
                    results[k] = True
            except (RuntimeError, OSError, ValueError) as e:
                err = str(e)
                self._maps.pop(int(nid), None)
        ok = all(results)
        return OpOutcome(ok, block_results=tuple(results), num_bytes=sum(results) * bb,
                         error="" if ok else f"{n - sum(results)} peer block(s) failed: {err}")


class PeerSsdWorker(TransferWorker):
    """PEERSSD2H: reads blocks that only another node's SSD tier holds straight out of that node's block files
    into this node's host pool. The owner published its file list and geometry in the registry; files are
    opened once per owner through this node's own IO engine (io_uring / O_DIRECT where they allow it). The
    reference asks the owner over ZeroMQ to stage the block and reads the staging buffer with RDMA
    (flexkv/transfer/worker.py:2920-3873); on one box, or over a shared mount, the files themselves are
    reachable. The owner's lease keeps the blocks in place while they are read."""

    name = "peerssd2h"

    def __init__(self, storage, registry) -> None:
        super().__init__()
        self.storage, self.registry = storage, registry
        self._engines: Dict[int, Tuple[Any, int]] = {}

    def _engine_of(self, nid: int):
        ent = self._engines.get(nid)
        if ent is not None:
            return ent
        import json
        meta = self.registry.get_node_meta(nid)
        if not meta or not meta.get("ssd_files"):
            raise RuntimeError(f"node {nid} has no SSD tier in the registry")
        st = self.storage
        mine = json.dumps(st.ssd_layout_dict(), sort_keys=True)
        if int(meta["ssd_block_bytes"]) != st.ssd.block_bytes or str(meta.get("ssd_layout")) != mine or \
                meta.get("codec", "none") != st.host.quant:
            raise RuntimeError(f"node {nid} uses a different SSD block format")
        files = json.loads(meta["ssd_files"])
        env = GLOBAL_CONFIG_FROM_ENV
        eng = _native.C.SsdIoEngine(files, int(meta["ssd_block_bytes"]), int(meta["ssd_blocks_per_file"]),
                                    create=False, try_direct=True, iouring_entries=env.iouring_entries,
                                    num_threads=max(2, env.ssd_io_threads // 2))
        ent = (eng, int(meta["ssd_num_blocks"]))
        self._engines[nid] = ent
        return ent

    def execute(self, op: TransferOp) -> OpOutcome:
        src, dst, nids = op.src_block_ids, op.dst_block_ids, op.remote_node_ids
        if nids is None or len(nids) != len(src) or len(src) != len(dst):
            return OpOutcome(False, error="peer SSD op without owner ids")
        st = self.storage
        n = len(src)
        results = [False] * n
        err = ""
        src = np.asarray(src, dtype=np.int64)
        dst = np.asarray(dst, dtype=np.int64)
        owners = np.asarray(nids, dtype=np.int64)
        lay = st.ssd_layout_dict()
        for nid in np.unique(owners).tolist():
            sel = np.nonzero(owners == nid)[0]
            try:
                eng, nblk = self._engine_of(int(nid))
                s_ids = np.ascontiguousarray(src[sel])
                d_ids = np.ascontiguousarray(dst[sel])
                if s_ids.min() < 0 or s_ids.max() >= nblk:
                    raise RuntimeError(f"block {int(s_ids.max())} outside node {nid}'s SSD tier")
                if d_ids.min() < 0 or d_ids.max() >= st.host.num_blocks:
                    raise RuntimeError(f"destination block {int(d_ids.max())} outside the host pool")
                nfail, ok = eng.transfer(st.host.base, d_ids, s_ids, True, lay, 0, lay["num_layers"])
                for k, good in zip(sel.tolist(), ok):
                    results[k] = bool(good)
                if nfail:
                    err = f"{nfail} read(s) from node {nid}'s files failed"
            except (RuntimeError, OSError, ValueError) as e:
                err = str(e)
                self._engines.pop(int(nid), None)
        ok_all = all(results)
        return OpOutcome(ok_all, block_results=tuple(results), num_bytes=sum(results) * st.host.block_bytes,
                         error="" if ok_all else f"{n - sum(results)} peer SSD block(s) failed: {err}")

    def close(self) -> None:
        self._engines.clear()


_GDS_PROBE: Optional[Tuple[bool, str]] = None


def gds_probe(timeout_s: float = 30.0) -> Tuple[bool, str]:
    """Opens the cuFile driver in a child process first: on hosts without a working
    GPUDirect Storage stack the driver open may block for a long time, and a child can
    be abandoned where a call in this process cannot."""
    global _GDS_PROBE
    if _GDS_PROBE is not None:
        return _GDS_PROBE
    import subprocess
    import sys
    import tempfile
    code = ("import sys, os, tempfile\n"
            "sys.path.insert(0, %r)\n"
            "from flexkv_b200 import _native\n"
            "d = tempfile.mkdtemp()\n"
            "p = os.path.join(d, 'probe.bin')\n"
            "open(p, 'wb').truncate(1 << 20)\n"
            "e = _native.C.GdsEngine([[p]], 1 << 20, 1, 1)\n"
            "print('GDS_OK' if e.available else 'GDS_NO ' + e.why_unavailable)\n"
            ) % os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=timeout_s,
                             cwd=tempfile.gettempdir())
        if "GDS_OK" in out.stdout:
            _GDS_PROBE = (True, "")
        else:
            tail = (out.stdout.strip().splitlines() or out.stderr.strip().splitlines() or ["no output"])[-1]
            _GDS_PROBE = (False, tail[:200])
    except subprocess.TimeoutExpired:
        _GDS_PROBE = (False, f"cuFile driver open did not return within {timeout_s:.0f} s")
    except OSError as e:
        _GDS_PROBE = (False, str(e))
    return _GDS_PROBE


class GdsWorker(TransferWorker):
    """DISK2D / D2DISK: SSD blocks move to or from the paged GPU cache without
    passing through the host pool. With GPUDirect Storage (cuFile) a block is read
    straight into a device bounce buffer; otherwise it is staged through a small
    pinned buffer with O_DIRECT io_uring reads. Either way the scatter into the
    paged layout is the ordinary copy kernel with the bounce buffer as its flat side
    (flexkv/transfer/worker.py:1948-2244; csrc/gds/gds_manager.cpp:596-795)."""

    def __init__(self, storage, model_config: ModelConfig, key: WorkerKey, to_gpu: bool, slots: int = 64) -> None:
        super().__init__()
        import torch
        self._torch = torch
        self.to_gpu = to_gpu
        self.name = "disk2d" if to_gpu else "d2disk"
        self.storage = storage
        self.regs = [storage.gpu_regs[key][r] for r in sorted(storage.gpu_regs[key])]
        host = storage.host
        self.shared = model_config.use_mla or model_config.num_kv_heads == 1
        n = 1 if self.shared else model_config.effective_tp_size
        self.slice_bytes = host.block_bytes // n
        self.layer_stride, self.kv_stride = host.layer_stride // n, host.kv_stride // n
        self.slots = slots
        ssd = storage.ssd
        self.gds = None
        why = "disabled by FLEXKV_GDS_FORCE_STAGED"
        if os.environ.get("FLEXKV_GDS_FORCE_STAGED", "0") != "1":
            ok, why = gds_probe()
            if ok:
                self.gds = _native.C.GdsEngine(ssd.files, ssd.block_bytes, ssd.blocks_per_file,
                                               int(os.environ.get("FLEXKV_GDS_THREADS", 8)))
                if not self.gds.available:
                    why, self.gds = self.gds.why_unavailable, None
        self.direct = self.gds is not None
        if not self.direct:
            flexkv_logger.info("GDS direct path unavailable (%s): staging through pinned memory", why)
        self.bounce, self.streams, self.status = {}, {}, {}
        for reg in self.regs:
            dev = f"cuda:{reg.device_id}"
            self.bounce[reg.device_id] = torch.empty(slots * self.slice_bytes, dtype=torch.uint8, device=dev)
            self.streams[reg.device_id] = torch.cuda.Stream(device=reg.device_id)
            self.status[reg.device_id] = torch.zeros(8, dtype=torch.int32, device=dev)
            if self.direct:
                self.gds.register_buffer(self.bounce[reg.device_id].data_ptr(), slots * self.slice_bytes)
        self.stage = None if self.direct else torch.empty(slots * host.block_bytes, dtype=torch.uint8).pin_memory()
        self.slot_ids = torch.arange(slots, dtype=torch.int64).pin_memory()

    def _scatter(self, reg, gpu_ids, n: int, base_ptr: int, block_stride: int, off: int, h2d: bool) -> int:
        torch = self._torch
        g = torch.from_numpy(np.ascontiguousarray(gpu_ids, dtype=np.int64)).pin_memory()
        params = dict(gpu_ptrs=[int(p) for p in reg.ptrs], idx_layer_mul=reg.idx_layer_mul, idx_kv_mul=reg.idx_kv_mul,
                      g_layer_stride=reg.layer_stride, g_kv_stride=reg.kv_stride, g_block_stride=reg.block_stride,
                      cpu_base=base_ptr, c_layer_stride=self.layer_stride, c_kv_stride=self.kv_stride,
                      c_block_stride=block_stride, c_off=off, gpu_blocks_ptr=g.data_ptr(),
                      cpu_blocks_ptr=self.slot_ids.data_ptr(), num_pairs=n, layer_start=0, num_layers=reg.num_layers,
                      kv_dim=reg.kv_dim, chunk_bytes=reg.chunk_bytes, gpu_num_blocks=reg.num_blocks,
                      cpu_num_blocks=self.slots, status_ptr=self.status[reg.device_id].data_ptr(), h2d=int(h2d))
        st = self.streams[reg.device_id]
        with torch.cuda.device(reg.device_id):
            _native.C.kv_copy(params, 16, 16384, 0, st.cuda_stream)
            st.synchronize()
        words = self.status[reg.device_id].tolist()
        bad = sum(1 << b for b, w in enumerate(words) if w)
        if bad:
            self.status[reg.device_id].zero_()
        return bad

    def execute(self, op: TransferOp) -> OpOutcome:
        ssd_ids, gpu_ids = (op.src_block_ids, op.dst_block_ids) if self.to_gpu else (op.dst_block_ids, op.src_block_ids)
        if ssd_ids.size != gpu_ids.size:
            return OpOutcome(False, error="unbound GPU blocks")
        st = self.storage
        failed = np.zeros(ssd_ids.size, dtype=bool)
        status = 0
        for lo in range(0, int(ssd_ids.size), self.slots):
            s_chunk = np.ascontiguousarray(ssd_ids[lo:lo + self.slots], dtype=np.int64)
            g_chunk = gpu_ids[lo:lo + self.slots]
            n = int(s_chunk.size)
            if not self.direct:
                slot_ids = np.arange(n, dtype=np.int64)
                if self.to_gpu:
                    lay = dict(st.ssd_layout_dict(), cpu_block_stride=st.host.block_bytes)
                    nfail, ok = st.ssd.engine.transfer(self.stage.data_ptr(), slot_ids, s_chunk, True, lay, 0,
                                                       lay["num_layers"])
                    failed[lo:lo + n] |= ~ok.astype(bool)
            for i, reg in enumerate(self.regs):
                if self.shared and not self.to_gpu and i > 0:
                    break
                off = 0 if self.shared else i * self.slice_bytes
                if self.direct:
                    offs = np.arange(n, dtype=np.int64) * self.slice_bytes
                    base = self.bounce[reg.device_id].data_ptr()
                    if self.to_gpu:
                        nfail, ok = self.gds.transfer(base, offs, s_chunk, True, off, self.slice_bytes)
                        failed[lo:lo + n] |= ~ok.astype(bool)
                        status |= self._scatter(reg, g_chunk, n, base, self.slice_bytes, 0, True)
                    else:
                        status |= self._scatter(reg, g_chunk, n, base, self.slice_bytes, 0, False)
                        nfail, ok = self.gds.transfer(base, offs, s_chunk, False, off, self.slice_bytes)
                        failed[lo:lo + n] |= ~ok.astype(bool)
                else:
                    status |= self._scatter(reg, g_chunk, n, self.stage.data_ptr(), st.host.block_bytes, off,
                                            self.to_gpu)
            if not self.direct and not self.to_gpu:
                lay = dict(st.ssd_layout_dict(), cpu_block_stride=st.host.block_bytes)
                nfail, ok = st.ssd.engine.transfer(self.stage.data_ptr(), np.arange(n, dtype=np.int64), s_chunk, False,
                                                   lay, 0, lay["num_layers"])
                failed[lo:lo + n] |= ~ok.astype(bool)
        good = status == 0 and not failed.any()
        return OpOutcome(good, block_results=tuple(bool(x) for x in ~failed),
                         num_bytes=int((~failed).sum()) * st.ssd.block_bytes,
                         error="" if good else f"gds: status 0x{status:x}, {int(failed.sum())} block(s) failed")

    def close(self) -> None:
        if self.direct:
            for t in self.bounce.values():
                self.gds.deregister_buffer(t.data_ptr())


def build_workers(storage, model_config: ModelConfig, cache_config: CacheConfig
                  ) -> Dict[Tuple[WorkerKey, TransferType], TransferWorker]:
    workers: Dict[Tuple[WorkerKey, TransferType], TransferWorker] = {}
    for key, regs in storage.gpu_regs.items():
        reg0 = regs[sorted(regs)[0]]
        if storage.host.layout.is_multi_group:
            workers[(key, TransferType.H2D)] = MultiGroupGpuHostWorker(storage, model_config, key, True)
            workers[(key, TransferType.D2H)] = MultiGroupGpuHostWorker(storage, model_config, key, False)
            if GLOBAL_CONFIG_FROM_ENV.enable_layerwise_transfer and reg0.device_id >= 0:
                from .layerwise import LayerwiseWorker, build_layerwise_eventfd_socket_path
                workers[(key, TransferType.LAYERWISE)] = LayerwiseWorker(
                    storage, model_config, key,
                    sock_path=build_layerwise_eventfd_socket_path(key.dp_client_id, key.pp_rank, model_config))
            continue
        if reg0.device_id < 0:
            workers[(key, TransferType.H2D)] = HostEmulatedGpuWorker(storage, model_config, key, True)
            workers[(key, TransferType.D2H)] = HostEmulatedGpuWorker(storage, model_config, key, False)
            continue
        if storage.host.quant != "none":
            workers[(key, TransferType.H2D)] = QuantGpuHostWorker(storage, model_config, key, True)
            workers[(key, TransferType.D2H)] = QuantGpuHostWorker(storage, model_config, key, False)
            continue
        per_rank_block = reg0.num_layers * reg0.kv_dim * reg0.chunk_bytes
        shared = model_config.use_mla or model_config.num_kv_heads == 1
        fanout = shared and len(regs) == 1 and getattr(reg0, "mc_ptrs", None)
        if fanout:
            workers[(key, TransferType.H2D)] = NvlsFanoutWorker(storage, model_config, key)
        for h2d in ((False,) if fanout else (True, False)):
            # one native group (thread + stream per GPU) per direction: PCIe is full duplex, so an offload and a
            # restore that are in flight together must not queue behind each other on one stream
            group = build_transfer_group(storage, model_config, key)
            w = GpuHostWorker(group, h2d, per_rank_block, len(regs) if (h2d or not shared) else 1)
            w.group_layers = reg0.num_layers
            w.max_blocks = max(4096, min(1 << 18, storage.host.num_blocks))
            workers[(key, TransferType.H2D if h2d else TransferType.D2H)] = w
        if GLOBAL_CONFIG_FROM_ENV.enable_layerwise_transfer:
            from .layerwise import LayerwiseWorker, build_layerwise_eventfd_socket_path
            workers[(key, TransferType.LAYERWISE)] = LayerwiseWorker(
                storage, model_config, key,
                sock_path=build_layerwise_eventfd_socket_path(key.dp_client_id, key.pp_rank, model_config))
    for key in storage.swa_regs:
        workers[(key, "SWA")] = SwaWorker(storage, model_config, key)
    real = [k for k, regs in storage.gpu_regs.items() if regs[sorted(regs)[0]].device_id >= 0]
    if cache_config.enable_p2p_gpu and len(real) > 1:
        peer = PeerD2DWorker(storage, model_config)
        for k in real:
            workers[(k, TransferType.PEERD2D)] = peer
    if storage.ssd is not None and cache_config.enable_gds and storage.host.quant == "none":
        for k in real:
            workers[(k, TransferType.DISK2D)] = GdsWorker(storage, model_config, k, True)
            workers[(k, TransferType.D2DISK)] = GdsWorker(storage, model_config, k, False)
    if cache_config.enable_remote and storage.host is not None:
        from ..external.remote_store import get_backend
        backend = get_backend(cache_config, storage.host.block_bytes)
        if backend is not None:
            registry = None
            if cache_config.enable_3rd_remote and not backend.key_addressed:
                from ..cache.hie_cache_engine import get_node_registry
                registry = get_node_registry(cache_config, model_config)
            workers[(WorkerKey(0, 0), TransferType.REMOTE2H)] = RemoteWorker(storage, backend, True, registry)
            workers[(WorkerKey(0, 0), TransferType.H2REMOTE)] = RemoteWorker(storage, backend, False)
    if cache_config.enable_p2p_cpu and storage.host is not None:
        from ..cache.hie_cache_engine import get_node_registry
        workers[(WorkerKey(0, 0), TransferType.PEERH2H)] = PeerHostWorker(
            storage, get_node_registry(cache_config, model_config))
    if cache_config.enable_p2p_ssd and storage.ssd is not None and storage.host is not None:
        from ..cache.hie_cache_engine import get_node_registry
        workers[(WorkerKey(0, 0), TransferType.PEERSSD2H)] = PeerSsdWorker(
            storage, get_node_registry(cache_config, model_config))
    if storage.ssd is not None:
        k0 = WorkerKey(0, 0)
        workers[(k0, TransferType.DISK2H)] = SsdWorker(storage, True)
        workers[(k0, TransferType.H2DISK)] = SsdWorker(storage, False)
    return workers
