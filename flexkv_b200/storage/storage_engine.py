"""Tier storage: the host block pool, SSD cache files and GPU registrations.

Reference counterparts: flexkv/storage/storage_engine.py:40-492 and
flexkv/storage/allocator.py:190-690. The host pool is one native region
(hugepage or THP-backed, placed on the NUMA node of the owning GPU, registered
PORTABLE|MAPPED so kernels can address it); SSD files follow the reference's
naming and sizing so cache directories are interchangeable:
``{dir_d}/{prefix}_{d}_{j}.bin``, each pre-sized to
``num_blocks_per_file * block_bytes``, ``num_ssd_blocks % num_devices == 0``.
"""
from __future__ import annotations

import os
import shutil
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import _native
from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig, parse_path_list
from ..common.debug import flexkv_logger
from ..common.storage import GroupLayout, KVCacheLayout, KVCacheLayoutType
from ..common.transfer import WorkerKey
from .gpu_layout import GpuRegistration

QUANT_GROUP = 128     # values per fp32 scale of the block-scaled fp8 host format


COMPRESS_TILE_ELEMS = 8192
COMPRESS_TILE_SLOT = 2 * COMPRESS_TILE_ELEMS + 128


def packed_chunk_bytes(chunk_elems: int, quant: str, itemsize: int) -> int:
    """Bytes one chunk occupies on the host tier."""
    if quant == "bf16_xp":
        if chunk_elems % 1024:
            raise ValueError("the exponent-packing codec needs chunk elements divisible by 1024")
        full, rest = divmod(chunk_elems, COMPRESS_TILE_ELEMS)
        return full * COMPRESS_TILE_SLOT + ((2 * rest + 128) if rest else 0)
    if quant == "fp8_e4m3":
        if chunk_elems % QUANT_GROUP:
            raise ValueError("fp8 offload needs chunk elements divisible by 128")
        return chunk_elems + (chunk_elems // QUANT_GROUP) * 4
    return chunk_elems * itemsize


@dataclass
class HostPool:
    region: Any                 # native HostRegion
    layout: KVCacheLayout
    block_bytes: int
    layer_stride: int           # bytes
    kv_stride: int
    chunk_bytes: int            # bytes of one (layer, kv) chunk holding every rank's heads
    num_blocks: int
    quant: str = "none"         # host codec: none | fp8_e4m3 (lossy, block-scaled) | bf16_xp (lossless)
    size_table: Any = None      # bf16_xp: pinned int32 tensor, one entry per (block, layer, kv, tile)
    tiles_per_chunk: int = 1

    @property
    def base(self) -> int:
        return int(self.region.ptr)

    def as_numpy(self) -> np.ndarray:
        return np.frombuffer(self.region, dtype=np.uint8)[: self.num_blocks * self.block_bytes]

    def block_view(self, block_id: int) -> np.ndarray:
        return self.as_numpy()[block_id * self.block_bytes:(block_id + 1) * self.block_bytes]


@dataclass
class SwaPool:
    """Host side of the sliding-window pool: [slot][rank][layer][page bytes]."""
    region: Any
    num_slots: int
    slot_bytes: int             # all ranks
    rank_slot_bytes: int
    page_bytes: int             # one layer of one rank (window KV group)
    group_layers: List[int] = None          # per group inside a rank's slot: layers,
    group_page_bytes: List[int] = None      # bytes of one layer's page,
    group_offsets: List[int] = None         # and where the group starts

    @property
    def base(self) -> int:
        return int(self.region.ptr)


@dataclass
class SsdPool:
    engine: Any                 # native SsdIoEngine
    files: List[List[str]]
    block_bytes: int
    num_blocks: int
    blocks_per_file: int


def host_register_chunk_bytes() -> int:
    """Chunk size of the host pool's CUDA registration: FLEXKV_HOST_REGISTER_CHUNK_BYTES, or the reference's
    FLEXKV_CUDAHOST_CHUNK_SIZE_GB (flexkv/transfer/host_buffer.py:58); 0 registers the pool in one call."""
    v = os.environ.get("FLEXKV_HOST_REGISTER_CHUNK_BYTES")
    if v is not None:
        return max(0, int(v))
    gb = float(os.environ.get("FLEXKV_CUDAHOST_CHUNK_SIZE_GB", "0") or 0)
    return int(gb * (1 << 30)) if gb > 0 else 0


class StorageEngine:
    def __init__(self, model_config: ModelConfig, cache_config: CacheConfig, cuda_register: Optional[bool] = None,
                 numa_node: int = -1) -> None:
        self.model_config = model_config
        self.cache_config = cache_config
        self.env = GLOBAL_CONFIG_FROM_ENV
        self.gpu_regs: Dict[WorkerKey, Dict[int, GpuRegistration]] = {}
        self.host: Optional[HostPool] = None
        self.ssd: Optional[SsdPool] = None
        self.ssd_size_table: Optional[np.ndarray] = None
        self.swa_regs: Dict[WorkerKey, Dict[int, GpuRegistration]] = {}
        self.swa_group_regs: Dict[WorkerKey, Dict[int, Dict[int, GpuRegistration]]] = {}    # [key][rank][group]
        self.gpu_group_regs: Dict[WorkerKey, Dict[int, Dict[int, GpuRegistration]]] = {}
        self.swa_host: Optional[SwaPool] = None
        self.swa_ssd: Optional[SsdPool] = None
        self.swa_remote_path: str = ""          # remote window tier: a file of whole slots on the remote mount
        self.swa_remote_slots: int = 0
        self._cuda_register = torch.cuda.is_available() if cuda_register is None else cuda_register
        self._numa_node = numa_node
        if cache_config.enable_cpu:
            self._alloc_host()
        if cache_config.enable_ssd:
            self._alloc_ssd()

    # ---- host pool ----------------------------------------------------------------
    def _host_geometry(self) -> Tuple[int, int, int, int, KVCacheLayout]:
        m, c = self.model_config, self.cache_config
        T = c.tokens_per_block
        layers = m.num_layers_local
        if m.layer_groups:
            groups = []
            for g in m.layer_groups:
                dt = g.dtype or m.dtype
                heads_rank = g.num_kv_heads if g.num_kv_heads == 1 else g.num_kv_heads // m.effective_tp_size
                groups.append(GroupLayout(g.num_layers // m.pp_size, g.kv_dim, T // g.compress_ratio,
                                          max(1, heads_rank), g.head_size, dt.itemsize))
            slices = 1 if all(g.num_kv_heads == 1 for g in m.layer_groups) else m.effective_tp_size
            lay = KVCacheLayout(KVCacheLayoutType.BLOCKFIRST, layers, c.num_cpu_blocks, T, m.num_kv_heads,
                                m.head_size, is_mla=m.use_mla, groups=groups, tp_slices=slices)
            return lay.block_bytes_flat, 0, 0, 0, lay
        lay = KVCacheLayout(self.env.cpu_layout_type, layers, c.num_cpu_blocks, T, m.num_kv_heads, m.head_size,
                            is_mla=m.use_mla, kv_dim_override=m.kv_dim)
        self._codec = self._choose_codec(lay)
        slices = 1 if (m.use_mla or m.num_kv_heads == 1) else m.effective_tp_size
        # every rank's slice of a chunk is packed on its own, so the host chunk is `slices` packed slices
        chunk = slices * packed_chunk_bytes(lay.get_chunk_size() // slices, self._codec, m.dtype.itemsize)
        if lay.type == KVCacheLayoutType.BLOCKFIRST:
            kv_stride, layer_stride = chunk, lay.kv_dim * chunk
            block_bytes = layers * layer_stride
        elif lay.type == KVCacheLayoutType.LAYERFIRST:
            kv_stride = c.num_cpu_blocks * chunk
            layer_stride = lay.kv_dim * kv_stride
            block_bytes = chunk          # block stride
        else:
            kv_stride = chunk
            block_bytes = lay.kv_dim * chunk
            layer_stride = c.num_cpu_blocks * block_bytes
        return block_bytes, layer_stride, kv_stride, chunk, lay

    def _choose_codec(self, lay: KVCacheLayout) -> str:
        """fp8 when asked for; else the lossless codec when compression is on and the cache qualifies
        (bf16, BLOCKFIRST host layout, chunk elements % 1024 == 0, no layerwise restore: the layerwise
        kernel consumes raw host blocks — the reference applies the same all-or-nothing rule,
        flexkv/transfer/compression/ans/ans_utils.py:51-118)."""
        from ..transfer.compression.policy import choose_codec
        m, c = self.model_config, self.cache_config
        slices = 1 if (m.use_mla or m.num_kv_heads == 1) else m.effective_tp_size
        d = choose_codec(requested_quant=c.offload_quant,
                         compression_enabled=bool(c.enable_compression or self.env.enable_compression),
                         dtype=m.dtype, host_layout_type=lay.type, chunk_elems_per_rank=lay.get_chunk_size() // slices,
                         itemsize=m.dtype.itemsize, layerwise=bool(self.env.enable_layerwise_transfer),
                         peer_host_sharing=bool(c.enable_p2p_cpu or c.enable_p2p_ssd or c.enable_3rd_remote),
                         pipeline_stages=m.local_pp_stages)
        if d.reason:
            flexkv_logger.warning("host codec refused: %s; every tier runs uncompressed", d.reason)
        if d.warning:
            flexkv_logger.warning("%s", d.warning)
        return d.codec

    def _alloc_host(self) -> None:
        c = self.cache_config
        block_bytes, layer_stride, kv_stride, chunk, lay = self._host_geometry()
        total = self._host_total_bytes(block_bytes, lay)
        backing = os.environ.get("FLEXKV_HUGEPAGE_FILE", "") if c.use_hugepage_cpu_buffer else ""
        if c.use_hugepage_cpu_buffer and not backing and os.environ.get("FLEXKV_HUGETLBFS_DIR"):
            # the reference's spelling: a hugetlbfs mount, the pool is a file of its own in it
            # (flexkv/storage/allocator.py:262)
            backing = os.path.join(os.environ["FLEXKV_HUGETLBFS_DIR"], f"flexkv_host_{os.getpid()}")
        self._owned_backing = ""
        if (c.enable_p2p_cpu or os.environ.get("FLEXKV_HOST_POOL_SHM", "0") == "1") and not backing:
            # other nodes of the box map this pool to pull blocks out of it (FLEXKV_HOST_POOL_SHM=1 asks for the
            # same named shared-memory file without the cross-node index)
            import uuid
            backing = f"/dev/shm/flexkv_host_{os.getpid()}_{uuid.uuid4().hex[:8]}"
            self._owned_backing = backing
        self.host_backing_file = backing
        try:
            region = _native.C.host_region_alloc(total, hugepage=c.use_hugepage_cpu_buffer,
                                                 hugepage_bytes=c.hugepage_size_bytes, numa_node=self._numa_node,
                                                 populate=True, touch_threads=min(16, os.cpu_count() or 4),
                                                 cuda_register=self._cuda_register,
                                                 register_chunk_bytes=host_register_chunk_bytes(),
                                                 backing_file=backing)
        except RuntimeError as e:
            raise RuntimeError(f"host pool of {total / 2**30:.1f} GiB could not be allocated: {e}") from e
        self.host = HostPool(region, lay, block_bytes, layer_stride, kv_stride, chunk, c.num_cpu_blocks,
                             getattr(self, "_codec", c.offload_quant))
        if self.host.quant == "bf16_xp":
            m = self.model_config
            slices = 1 if (m.use_mla or m.num_kv_heads == 1) else m.effective_tp_size
            tpc = (lay.get_chunk_size() // slices + COMPRESS_TILE_ELEMS - 1) // COMPRESS_TILE_ELEMS
            self.host.tiles_per_chunk = tpc
            n = c.num_cpu_blocks * m.num_layers_local * lay.kv_dim * tpc * slices
            table = torch.zeros(n, dtype=torch.int32)
            self.host.size_table = table.pin_memory() if self._cuda_register else table
        flexkv_logger.info("host pool: %d blocks x %d B = %.2f GiB (hugepage=%s, registered=%s, layout=%s)",
                           c.num_cpu_blocks, block_bytes, total / 2**30, region.hugepage, region.registered,
                           lay.type.value)

    def _host_total_bytes(self, block_bytes: int, lay: KVCacheLayout) -> int:
        c = self.cache_config
        if lay.is_multi_group or lay.type == KVCacheLayoutType.BLOCKFIRST:
            return c.num_cpu_blocks * block_bytes
        return self.model_config.num_layers_local * lay.kv_dim * c.num_cpu_blocks * \
            packed_chunk_bytes(lay.get_chunk_size(), getattr(self, "_codec", c.offload_quant),
                               self.model_config.dtype.itemsize)

    def pp_stage_offset(self, pp_rank: int) -> int:
        """Byte offset of pipeline stage ``pp_rank``'s first layer inside the host pool's layer axis
        (stages served by this manager share one host block: stage s owns layers [s*Lp, (s+1)*Lp))."""
        m = self.model_config
        if m.local_pp_stages <= 1 or pp_rank <= 0:
            return 0
        return pp_rank * m.num_layers_per_pp_stage * self.host.layer_stride

    def host_block_stride(self) -> int:
        return self.host.block_bytes

    # ---- SSD ----------------------------------------------------------------------
    def _alloc_ssd(self) -> None:
        c = self.cache_config
        dirs = parse_path_list(c.ssd_cache_dir or [])
        if not dirs:
            raise ValueError("enable_ssd requires ssd_cache_dir")
        ndev = len(dirs)
        if c.num_ssd_blocks % ndev:
            raise ValueError(f"num_ssd_blocks ({c.num_ssd_blocks}) must be a multiple of the number of "
                             f"SSD directories ({ndev})")
        if self.host is None:
            raise ValueError("the SSD tier needs the host tier as staging")
        block_bytes = self.host.block_bytes if self.host.layout.type == KVCacheLayoutType.BLOCKFIRST or \
            self.host.layout.is_multi_group else \
            self.model_config.num_layers_local * self.host.layout.kv_dim * self.host.chunk_bytes
        per_dev = c.num_ssd_blocks // ndev
        max_gb = self.env.max_file_size_gb
        blocks_per_file = per_dev
        from ..cache import persist
        self._ssd_persist = persist.persist_enabled(c)
        for di, d in enumerate(dirs):
            os.makedirs(d, exist_ok=True)
            free = shutil.disk_usage(d).free
            if self._ssd_persist:
                # the files of the previous run are this tier's own space: the split into files
                # (and with it the place of every block) must come out the same again
                for name in os.listdir(d):
                    if name.startswith(f"flexkv_ssd_cache_{di}_") and name.endswith(".bin"):
                        free += os.stat(os.path.join(d, name)).st_blocks * 512
            blocks_per_file = min(blocks_per_file, max(1, free // block_bytes))
        if max_gb and max_gb > 0:
            blocks_per_file = min(blocks_per_file, max(1, int(max_gb * 2**30) // block_bytes))
        files_per_dev = (per_dev + blocks_per_file - 1) // blocks_per_file
        # a persistent tier keeps fixed file names so that the next process finds its blocks
        prefix = f"flexkv_ssd_cache_{os.getpid()}" if not self._ssd_persist and \
            os.environ.get("FLEXKV_SSD_FILE_PER_PROCESS", "1") == "1" else "flexkv_ssd_cache"
        files = [[os.path.join(d, f"{prefix}_{di}_{j}.bin") for j in range(files_per_dev)]
                 for di, d in enumerate(dirs)]
        engine = _native.C.SsdIoEngine(files, block_bytes, blocks_per_file, create=True, try_direct=True,
                                       iouring_entries=self.env.iouring_entries,
                                       num_threads=self.env.ssd_io_threads)
        self.ssd = SsdPool(engine, files, block_bytes, c.num_ssd_blocks, blocks_per_file)
        if self.host.size_table is not None:
            per_block = self.host.size_table.numel() // self.host.num_blocks
            self.ssd_size_table = np.zeros((c.num_ssd_blocks, per_block), dtype=np.int32)
            if self._ssd_persist and persist.load_size_table(c, self.ssd_size_table):
                flexkv_logger.info("ssd size table loaded from the previous run")
        flexkv_logger.info("ssd pool: %d blocks x %d B over %d dir(s), %d file(s)/dir, io_uring=%s direct=%s",
                           c.num_ssd_blocks, block_bytes, ndev, files_per_dev, engine.using_iouring,
                           engine.direct_available)

    def packed_ssd_geometry(self) -> Optional[Dict[str, int]]:
        """Tile-slot geometry of a host block for packed SSD IO, or None when the pool is not in the lossless
        codec's format (or ``FLEXKV_SSD_PACKED=0``): the SSD then moves whole slots."""
        if self.ssd is None or self.ssd_size_table is None or self.host.size_table is None:
            return None
        if os.environ.get("FLEXKV_SSD_PACKED", "1") == "0":
            return None
        tpc = int(self.host.tiles_per_chunk)
        entries = int(self.ssd_size_table.shape[1])
        # a rank's chunk slot: the block is [rank slice][layer][kv][slot], the table row walks it in that order
        chunk_slot = int(self.host.chunk_bytes) // max(1, int(getattr(self.host.layout, "tp_slices", 1)))
        last = chunk_slot - (tpc - 1) * COMPRESS_TILE_SLOT
        return dict(cpu_block_stride=int(self.host.block_bytes), chunk_slot_bytes=chunk_slot,
                    tile_slot_bytes=COMPRESS_TILE_SLOT, last_tile_slot_bytes=int(last), tiles_per_chunk=tpc,
                    entries=entries)

    def sync_ssd_files(self) -> None:
        """fsync of every SSD block file and of the directories that hold them (a persisted index must not
        name blocks that only exist in the page cache)."""
        if self.ssd is None:
            return
        try:
            self.ssd.engine.sync_files()
        except Exception as e:  # noqa: BLE001
            flexkv_logger.warning("ssd block files not synced: %s", e)
        for d in {os.path.dirname(os.path.abspath(f)) for dev in self.ssd.files for f in dev}:
            try:
                fd = os.open(d, os.O_RDONLY | os.O_DIRECTORY)
                try:
                    os.fsync(fd)
                finally:
                    os.close(fd)
            except OSError:
                pass

    def ssd_layout_dict(self) -> Dict[str, Any]:
        h = self.host
        bf = h.layout.type == KVCacheLayoutType.BLOCKFIRST or h.layout.is_multi_group
        L = self.model_config.num_layers_local
        if bf:
            ssd_layer, ssd_kv = h.layer_stride, h.kv_stride
        else:
            ssd_kv = h.chunk_bytes
            ssd_layer = h.layout.kv_dim * h.chunk_bytes
        if h.layout.is_multi_group:
            # one run per block: describe the block as a single "layer"
            return dict(cpu_layer_stride=h.block_bytes, cpu_kv_stride=0, cpu_block_stride=h.block_bytes,
                        ssd_layer_stride=h.block_bytes, ssd_kv_stride=0, ssd_block_stride=h.block_bytes,
                        chunk_bytes=h.block_bytes, num_layers=1, kv_dim=1, block_first=True)
        return dict(cpu_layer_stride=h.layer_stride, cpu_kv_stride=h.kv_stride, cpu_block_stride=h.block_bytes,
                    ssd_layer_stride=ssd_layer, ssd_kv_stride=ssd_kv, ssd_block_stride=self.ssd.block_bytes,
                    chunk_bytes=h.chunk_bytes, num_layers=L, kv_dim=h.layout.kv_dim, block_first=bf)

    def swa_ssd_layout_dict(self) -> Dict[str, Any]:
        """A window slot is one run of bytes on both sides."""
        b = self.swa_ssd.block_bytes
        return dict(cpu_layer_stride=b, cpu_kv_stride=0, cpu_block_stride=b, ssd_layer_stride=b, ssd_kv_stride=0,
                    ssd_block_stride=b, chunk_bytes=b, num_layers=1, kv_dim=1, block_first=True)

    # ---- sliding-window side pool ------------------------------------------------------
    def register_swa_blocks(self, reg: GpuRegistration) -> None:
        """GPU window pages of one rank: ``num_layers`` tensors of [pages, page_bytes]. ``group_id``
        0 (or -1) is the window KV itself, g >= 1 the g-th sidecar group of ``SWAPoolConfig.sidecar_groups``
        (state that is saved and restored with the same slot)."""
        key = WorkerKey(reg.dp_client_id, reg.pp_rank)
        g = max(0, int(reg.group_id))
        if self.swa_host is None:
            self._alloc_swa(reg if g == 0 else None)
        pool = self.swa_host
        if g >= len(pool.group_layers):
            raise ValueError(f"window sidecar group {g} is not configured (SWAPoolConfig.sidecar_groups)")
        if (reg.num_layers, reg.chunk_bytes) != (pool.group_layers[g], pool.group_page_bytes[g]):
            raise ValueError(f"window group {g}: registered {reg.num_layers} layers x {reg.chunk_bytes} B, the pool "
                             f"expects {pool.group_layers[g]} x {pool.group_page_bytes[g]} B")
        self.swa_group_regs.setdefault(key, {}).setdefault(reg.tp_rank, {})[g] = reg
        if g == 0:
            self.swa_regs.setdefault(key, {})[reg.tp_rank] = reg

    def _alloc_swa(self, reg: Optional[GpuRegistration]) -> None:
        cfg = self.cache_config.swa
        if cfg is None or not cfg.enabled:
            raise ValueError("window pages registered but CacheConfig.swa is not enabled")
        ranks = 1 if (self.model_config.use_mla or self.model_config.num_kv_heads == 1) else \
            self.model_config.effective_tp_size
        geometry = cfg.group_geometry(self.cache_config.tokens_per_block)
        if reg is not None and not cfg.sidecar_groups:
            geometry = [(reg.num_layers, reg.chunk_bytes)]      # a lone window group is sized by its tensors
        layers = [n for n, _ in geometry]
        pages = [b for _, b in geometry]
        offsets = [0]
        for n, b in geometry[:-1]:
            offsets.append(offsets[-1] + n * b)
        rank_slot = sum(n * b for n, b in geometry)
        total = cfg.num_slots * ranks * rank_slot
        region = _native.C.host_region_alloc(total, hugepage=False, hugepage_bytes=2 << 20, numa_node=self._numa_node,
                                             populate=True, touch_threads=4,
                                             cuda_register=self._cuda_register and cfg.pin_memory,
                                             register_chunk_bytes=0, backing_file="")
        self.swa_host = SwaPool(region, cfg.num_slots, ranks * rank_slot, rank_slot, pages[0], layers, pages, offsets)
        if cfg.num_ssd_slots > 0 and self.cache_config.enable_ssd:
            # SSD window tier: one file of whole slots in the first cache directory
            d = parse_path_list(self.cache_config.ssd_cache_dir or [])[0]
            os.makedirs(d, exist_ok=True)
            path = os.path.join(d, f"flexkv_swa_cache_{os.getpid()}.bin")
            engine = _native.C.SsdIoEngine([[path]], ranks * rank_slot, cfg.num_ssd_slots, create=True,
                                           try_direct=True, iouring_entries=self.env.iouring_entries,
                                           num_threads=2)
            self.swa_ssd = SsdPool(engine, [[path]], ranks * rank_slot, cfg.num_ssd_slots, cfg.num_ssd_slots)
        if cfg.num_remote_slots > 0 and self.cache_config.enable_remote and self.cache_config.remote_cache_path:
            # remote window tier: one file of whole slots on the remote mount, plain positional IO
            d = parse_path_list(self.cache_config.remote_cache_path)[0]
            os.makedirs(d, exist_ok=True)
            self.swa_remote_path = os.path.join(
                d, f"{self.cache_config.remote_file_prefix or 'flexkv_remote'}_swa.bin")
            with open(self.swa_remote_path, "ab") as f:
                f.truncate(cfg.num_remote_slots * ranks * rank_slot)
            self.swa_remote_slots = cfg.num_remote_slots
        flexkv_logger.info("window pool: %d slots x %d B (groups of layers x page bytes per rank: %s, %d rank(s))",
                           cfg.num_slots, ranks * rank_slot, geometry, ranks)

    def register_gpu_blocks(self, reg: GpuRegistration) -> None:
        key = WorkerKey(reg.dp_client_id, reg.pp_rank)
        if reg.group_id >= 0:
            # multi-group cache: one registration per (rank, layer group); the first group also stands
            # for the rank in the per-rank table
            self.gpu_group_regs.setdefault(key, {}).setdefault(reg.tp_rank, {})[reg.group_id] = reg
            self.gpu_regs.setdefault(key, {}).setdefault(reg.tp_rank, reg)
            return
        self.gpu_regs.setdefault(key, {})[reg.tp_rank] = reg

    def all_registered(self) -> bool:
        m = self.model_config
        want_keys = m.total_clients * m.local_pp_stages
        if len(self.gpu_regs) < want_keys:
            return False
        return all(len(r) >= m.effective_tp_size_per_node for r in self.gpu_regs.values())

    def close_gpu_mappings(self) -> None:
        """Drops this process's view of every registered cache that was opened from a handle (CUDA IPC or
        virtual-memory handles of another process). The owner may free its cache as soon as the manager is shut
        down; freeing exported memory that an importer still maps is undefined behaviour in CUDA."""
        seen = set()
        regs = [r for ranks in self.gpu_regs.values() for r in ranks.values()]
        regs += [g for per_rank in self.gpu_group_regs.values() for per in per_rank.values() for g in per.values()]
        regs += [r for ranks in getattr(self, "swa_regs", {}).values()
                 for r in (ranks.values() if isinstance(ranks, dict) else ranks)]
        for reg in regs:
            keep = getattr(reg, "keepalive", None)
            for h in (keep if isinstance(keep, (list, tuple)) else [keep]):
                if h is not None and hasattr(h, "close") and id(h) not in seen:
                    seen.add(id(h))
                    try:
                        h.close()
                    except Exception:  # noqa: BLE001
                        pass

    def shutdown(self) -> None:
        self.close_gpu_mappings()
        if self.host is not None:
            try:
                self.host.region.free()
            except Exception:  # noqa: BLE001
                pass
            self.host = None
            if getattr(self, "_owned_backing", ""):
                try:
                    os.unlink(self._owned_backing)
                except OSError:
                    pass
        if self.swa_host is not None:
            try:
                self.swa_host.region.free()
            except Exception:  # noqa: BLE001
                pass
            self.swa_host = None
        if self.swa_ssd is not None:
            files = [f for d in self.swa_ssd.files for f in d]
            self.swa_ssd = None
            for f in files:
                try:
                    os.unlink(f)
                except OSError:
                    pass
        if self.ssd is not None:
            files = [f for d in self.ssd.files for f in d]
            if getattr(self, "_ssd_persist", False):
                self.sync_ssd_files()      # the index written after this names only bytes that reached the disk
            self.ssd = None
            if getattr(self, "_ssd_persist", False):
                from ..cache import persist
                persist.save_size_table(self.cache_config, self.ssd_size_table)
            elif os.environ.get("FLEXKV_KEEP_SSD_FILES", "0") != "1":
                for f in files:
                    try:
                        os.unlink(f)
                    except OSError:
                        pass
