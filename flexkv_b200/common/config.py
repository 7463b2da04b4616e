"""Configuration: model/cache dataclasses, the ``FLEXKV_*`` environment table,
user config files and GB -> block conversion.

Field and variable names match the reference so that existing deployments can
switch without renaming anything (flexkv/common/config.py:122-427 ModelConfig,
:430-571 RankInfo, :623-746 CacheConfig, :748-841 environment table,
:843-944 UserConfig, :946-1246 conversion helpers). GPU<->host moves default to one
sm_100a kernel per op; the copy-engine switches select the adaptive router that
sends long contiguous runs to the DMA engines instead.
"""
from __future__ import annotations

import json
import os
from argparse import Namespace
from dataclasses import replace, dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from .storage import KVCacheLayoutType

_DTYPE_ALIASES = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
    "half": torch.float16, "fp32": torch.float32, "float32": torch.float32, "float": torch.float32,
    "fp8": torch.float8_e4m3fn, "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2,
    "uint8": torch.uint8, "int8": torch.int8,
    # byte-exact NVFP4: the packed cache is moved as bytes, never interpreted
    "nvfp4": torch.uint8, "fp4": torch.uint8, "e2m1": torch.uint8, "fp4_e2m1": torch.uint8,
}
NVFP4_NAMES = ("nvfp4", "fp4", "e2m1", "fp4_e2m1")


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).lower().replace("torch.", "")
    if key not in _DTYPE_ALIASES:
        raise ValueError(f"unsupported kv cache dtype: {name}")
    return _DTYPE_ALIASES[key]


def nvfp4_head_bytes(head_size: int) -> int:
    """Bytes per token per head of a packed NVFP4 cache: e2m1 nibbles plus one
    e4m3 scale per 16 elements (flexkv/integration/config.py:24-36,142-150)."""
    return head_size // 2 + head_size // 16


@dataclass
class LayerGroupSpec:
    """A run of layers with its own KV shape (e.g. an indexer or a compressed-KV group)."""
    num_layers: int
    num_kv_heads: int
    head_size: int
    kv_dim: int = 2
    dtype: Optional[torch.dtype] = None
    compress_ratio: int = 1           # tokens stored per block = tokens_per_block / ratio
    layer_ids: Optional[List[int]] = None
    name: str = ""
    layer_indices: Optional[List[int]] = None     # the reference's name for layer_ids; either may be given

    def __post_init__(self) -> None:
        if self.layer_ids is None and self.layer_indices is not None:
            self.layer_ids = list(self.layer_indices)
        elif self.layer_indices is None and self.layer_ids is not None:
            self.layer_indices = list(self.layer_ids)


@dataclass
class ModelConfig:
    num_layers: int = 1
    num_kv_heads: int = 1
    head_size: int = 1
    kv_dim: int = 2
    dtype: torch.dtype = torch.bfloat16
    use_mla: bool = False
    tp_size: int = 1
    pp_size: int = 1
    dp_size: int = 1
    enable_dp_attention: bool = False
    attn_cp_size: int = 1
    cp_size: int = 1
    nnodes: int = 1
    master_host: str = "localhost"
    master_ports: Tuple[str, str, str] = ("5556", "5557", "5558")
    use_trtllm_subprocess: bool = False
    trtllm_subprocess_host: str = "localhost"
    trtllm_subprocess_ports: Tuple[str, str, str] = ("6667", "6668", "6669")
    instance_num: int = 1
    layer_groups: Optional[List[LayerGroupSpec]] = None
    _frozen: bool = field(default=False, init=False, repr=False, compare=False)

    def __post_init__(self) -> None:
        if self.use_mla:
            object.__setattr__(self, "kv_dim", 1)
        elif self.kv_dim == 1 and self.num_kv_heads == 1:
            object.__setattr__(self, "use_mla", True)

    def __setattr__(self, name: str, value: Any) -> None:
        if getattr(self, "_frozen", False) and name != "_frozen":
            raise AttributeError(f"ModelConfig is frozen; cannot set {name}")
        object.__setattr__(self, name, value)

    def freeze(self) -> None:
        if self.cp_size == 1 and self.attn_cp_size != 1:
            self.cp_size = self.attn_cp_size
        elif self.attn_cp_size == 1 and self.cp_size != 1:
            self.attn_cp_size = self.cp_size
        elif self.cp_size != self.attn_cp_size:
            raise ValueError("cp_size and attn_cp_size disagree")
        if self.nnodes < 1 or self.total_gpus % self.nnodes:
            raise ValueError("total GPUs must divide evenly over nnodes")
        self._validate_layer_groups()
        object.__setattr__(self, "_frozen", True)

    def _validate_layer_groups(self) -> None:
        if not self.layer_groups:
            return
        for g in self.layer_groups:
            if g.num_layers <= 0 or g.head_size <= 0 or g.num_kv_heads <= 0:
                raise ValueError(f"bad layer group {g}")
            if g.compress_ratio < 1:
                raise ValueError("compress_ratio must be >= 1")

    # ---- topology -------------------------------------------------------------
    @property
    def total_gpus(self) -> int:
        return self.tp_size * self.cp_size * self.pp_size * self.dp_size

    @property
    def total_clients(self) -> int:
        return self.dp_size * self.instance_num

    @property
    def gpus_per_node(self) -> int:
        return max(1, self.total_gpus // self.nnodes)

    @property
    def effective_tp_size(self) -> int:
        """Slices of one host block: every (cp_rank, tp_rank) pair owns one."""
        return self.tp_size * self.cp_size

    @property
    def nnodes_per_tp_group(self) -> int:
        return max(1, (self.effective_tp_size + self.gpus_per_node - 1) // self.gpus_per_node)

    @property
    def effective_tp_size_per_node(self) -> int:
        return self.effective_tp_size // self.nnodes_per_tp_group

    @property
    def tp_size_per_node(self) -> int:
        return max(1, self.tp_size // self.nnodes_per_tp_group)

    @property
    def num_layers_per_pp_stage(self) -> int:
        return self.num_layers // self.pp_size

    @property
    def local_pp_stages(self) -> int:
        """Pipeline stages whose GPUs one manager serves: all of them on a single node (their layers share
        one host block, stage s at layer offset s * layers_per_stage); one per node otherwise."""
        return self.pp_size if self.nnodes == 1 else 1

    @property
    def num_layers_local(self) -> int:
        return self.num_layers_per_pp_stage * self.local_pp_stages

    # ---- sizes ----------------------------------------------------------------
    @property
    def bytes_per_token_per_layer(self) -> int:
        return self.kv_dim * self.num_kv_heads * self.head_size * self.dtype.itemsize

    @property
    def token_size_in_bytes(self) -> int:
        """Bytes of KV one token occupies across all layers (all TP ranks together)."""
        if self.layer_groups:
            total = 0
            for g in self.layer_groups:
                dt = g.dtype or self.dtype
                total += g.num_layers * g.kv_dim * g.num_kv_heads * g.head_size * dt.itemsize // g.compress_ratio
            return total
        return self.num_layers * self.bytes_per_token_per_layer

    @property
    def token_size_in_bytes_per_pp_stage(self) -> int:
        return self.token_size_in_bytes // self.pp_size

    def block_size_in_bytes(self, tokens_per_block: int) -> int:
        if self.layer_groups:
            total = 0
            for g in self.layer_groups:
                dt = g.dtype or self.dtype
                total += g.num_layers * g.kv_dim * (tokens_per_block // g.compress_ratio) * g.num_kv_heads \
                    * g.head_size * dt.itemsize
            return total
        return self.token_size_in_bytes * tokens_per_block


@dataclass
class RankInfo:
    """Where one engine worker sits in the tp x cp x pp x dp grid
    (flexkv/common/config.py:430-571)."""
    model_config: ModelConfig
    tp_rank: int = 0
    cp_rank: int = 0
    pp_rank: int = 0
    dp_rank: int = 0
    instance_id: int = 0
    node_rank: int = 0
    device_id: int = 0
    # names the SGLang-facing callers of the reference use (flexkv/common/config.py:431-478)
    attn_cp_rank: int = 0            # mirror of cp_rank
    pp_start_layer: int = 0
    pp_end_layer: int = -1
    local_rank: int = -1             # GPU index on the node; derived from the ranks when negative

    def __post_init__(self) -> None:
        if self.cp_rank == 0 and self.attn_cp_rank != 0:
            self.cp_rank = self.attn_cp_rank
        elif self.attn_cp_rank == 0 and self.cp_rank != 0:
            self.attn_cp_rank = self.cp_rank
        elif self.cp_rank != self.attn_cp_rank:
            raise ValueError(f"cp_rank={self.cp_rank} and attn_cp_rank={self.attn_cp_rank} disagree")
        if self.local_rank < 0:
            m = self.model_config
            nn = max(1, getattr(m, "nnodes", 1))
            tp_node = max(1, m.tp_size_per_node)
            cp_node = max(1, getattr(m, "cp_size", 1))
            pp_node = max(1, m.local_pp_stages)
            tp_cp = self.cp_rank * tp_node + self.tp_rank % tp_node
            pp_local = self.pp_rank % pp_node
            if m.enable_dp_attention:
                self.local_rank = pp_local * cp_node * tp_node + tp_cp
            else:
                dp_node = max(1, m.dp_size // nn) if m.dp_size >= nn else 1
                self.local_rank = ((self.dp_rank % dp_node) * pp_node + pp_local) * cp_node * tp_node + tp_cp

    @property
    def attn_tp_rank(self) -> int:
        return self.tp_rank

    @property
    def dp_client_id(self) -> int:
        return self.instance_id * self.model_config.dp_size + self.dp_rank

    @property
    def effective_tp_rank(self) -> int:
        return self.cp_rank * self.model_config.tp_size + self.tp_rank

    @property
    def intra_client_id(self) -> int:
        m = self.model_config
        return self.pp_rank * m.effective_tp_size + self.effective_tp_rank


@dataclass
class SWAPoolConfig:
    """Sliding-window side pool: one slot holds the window state of one cache page
    (``tokens_per_block`` tokens) for every sliding-window layer
    (reference: flexkv/common/config.py:573-620)."""
    enabled: bool = False
    num_slots: int = 1024              # host slots
    num_ssd_slots: int = 0             # SSD window tier (0 = none): snapshots written through beside the SSD blocks
    num_remote_slots: int = 0          # remote window tier (0 = none), for the block-addressed remote tier
    num_swa_layers: int = 61
    bytes_per_token_per_layer: int = 584
    multi_group: bool = False
    evict_ratio: float = 0.1           # share of the pool freed when it runs full
    pin_memory: bool = True
    # state that rides in the same slot as the window KV (e.g. compressor states of an indexer): one
    # (num_layers, page_bytes_per_layer) pair per sidecar group; the group's tensors are registered with
    # group_id = 1 + its position here
    sidecar_groups: List[Tuple[int, int]] = field(default_factory=list)
    # engine ranks register their window pages from other processes: start-up waits for all of them
    wait_for_registration: bool = False

    def page_bytes_per_layer(self, tokens_per_block: int) -> int:
        return int(tokens_per_block) * int(self.bytes_per_token_per_layer)

    def slot_bytes(self, tokens_per_block: int) -> int:
        return sum(n * b for n, b in self.group_geometry(tokens_per_block))

    def group_geometry(self, tokens_per_block: int) -> List[Tuple[int, int]]:
        """(layers, page bytes per layer) of the window KV followed by the sidecar groups."""
        return [(int(self.num_swa_layers), self.page_bytes_per_layer(tokens_per_block))] + \
            [(int(n), int(b)) for n, b in self.sidecar_groups]

    def for_cache_tier(self, device_type) -> Optional["SWAPoolConfig"]:
        name = getattr(device_type, "name", str(device_type))
        if not self.enabled:
            return None
        if name == "CPU":
            return self
        if name == "SSD" and self.num_ssd_slots > 0:
            return replace(self, num_slots=self.num_ssd_slots, pin_memory=False)
        if name == "REMOTE" and self.num_remote_slots > 0:
            return replace(self, num_slots=self.num_remote_slots, pin_memory=False)
        return None


@dataclass
class CacheConfig:
    tokens_per_block: int = 16
    eviction_policy: str = "lru"
    enable_cpu: bool = True
    enable_ssd: bool = False
    enable_gds: bool = False
    enable_nixl: bool = False
    nixl_extra_config: Optional[Dict[str, Any]] = None
    enable_remote: bool = False
    enable_kv_sharing: bool = False
    enable_p2p_cpu: bool = False
    enable_p2p_ssd: bool = False
    enable_3rd_remote: bool = False
    # B200-native additions: cross-GPU prefix reuse over NVLink and quantised offload
    enable_p2p_gpu: bool = False
    offload_quant: str = "none"            # none | fp8_e4m3 (block-scaled, 1 fp32 scale / 128 values)
    enable_compression: bool = False       # lossless exponent-packing codec on the host tier
    distributed_node_id: int = -1
    num_tmp_cpu_blocks: int = 500
    use_hugepage_cpu_buffer: bool = False
    use_hugepage_tmp_buffer: bool = False
    hugepage_size_bytes: int = 2 * 1024 * 1024
    num_cpu_blocks: int = 1000000
    num_ssd_blocks: int = 10000000
    num_remote_blocks: Optional[int] = None
    num_local_blocks: int = 1000000
    ssd_cache_dir: Optional[Union[str, List[str]]] = None
    ssd_persist: bool = False              # keep the SSD files and their index across restarts (FLEXKV_SSD_PERSIST)
    remote_cache_size_mode: str = "file_size"
    remote_file_size: Optional[int] = None
    remote_file_num: Optional[int] = None
    remote_file_prefix: Optional[str] = None
    remote_cache_path: Optional[Union[str, List[str]]] = None
    remote_config_custom: Optional[Dict[str, Any]] = None
    local_zmq_ip: str = "127.0.0.1"
    local_zmq_port: int = 5555
    redis_host: str = "127.0.0.1"
    redis_port: int = 6379
    local_ip: str = "127.0.0.1"
    redis_password: Optional[str] = None
    node_ttl_seconds: int = 30
    mooncake_config_path: Optional[str] = None
    use_mooncake_store_backend: bool = False
    mooncake_store_config_path: Optional[str] = None
    mooncake_store_pp_rank: int = 0                # accepted for compatibility (no Mooncake library here)
    mooncake_store_pp_size: int = 1
    mooncake_store_node_layer_start: int = 0
    mooncake_store_node_layer_end: int = 0
    mooncake_store_total_layers: int = 0
    _user_cpu_cache_gb: float = 0
    _user_ssd_cache_gb: float = 0
    _swa_multi_group: Optional[bool] = None       # user switch: False leaves state sidecars out of the window slot
    swa: Optional[SWAPoolConfig] = None
    enable_swa_transfer: bool = False

    def __post_init__(self) -> None:
        if self.tokens_per_block <= 0 or self.tokens_per_block & (self.tokens_per_block - 1):
            raise ValueError("tokens_per_block must be a power of two")
        self.enable_kv_sharing = self.enable_p2p_cpu or self.enable_p2p_ssd or self.enable_3rd_remote
        self.enable_remote = self.enable_remote or self.enable_3rd_remote or self.use_mooncake_store_backend
        if self.enable_gds and not self.enable_ssd:
            raise ValueError("enable_gds requires enable_ssd")
        if self.offload_quant not in ("none", "fp8_e4m3"):
            raise ValueError(f"unknown offload_quant {self.offload_quant}")
        if self.enable_nixl and self.enable_ssd and not self.enable_gds:
            # NIXL's role here (SSD <-> GPU without the host pool) is the GDS worker's
            self.enable_gds = True

    def settings_without_effect(self) -> List[Tuple[str, str]]:
        """Fields kept for compatibility with the reference's configuration that do nothing in this build when
        set away from their defaults, each with the reason; the manager logs them at start-up so that a
        deployment file written for the reference does not fail silently."""
        out: List[Tuple[str, str]] = []
        if self.enable_nixl:
            out.append(("enable_nixl", "no NIXL library in this build: SSD <-> GPU ops run through the GDS worker "
                                       "(cuFile when it opens, else a pinned bounce buffer)"
                        if self.enable_ssd else "needs enable_ssd; no NIXL library in this build"))
        if self.nixl_extra_config:
            out.append(("nixl_extra_config", "no NIXL library in this build"))
        if self.use_hugepage_tmp_buffer or self.num_tmp_cpu_blocks != 500:
            out.append(("use_hugepage_tmp_buffer / num_tmp_cpu_blocks",
                        "peer reads land in blocks of the host pool itself; there is no separate staging buffer"))
        if self.mooncake_config_path or self.mooncake_store_config_path:
            out.append(("mooncake_config_path / mooncake_store_config_path",
                        "no Mooncake library in this build: peer reads map the owner's pool or block files, the "
                        "key-addressed store is remote_config_custom"))
        if self.enable_3rd_remote and self.use_mooncake_store_backend:
            out.append(("enable_3rd_remote", "a key-addressed store is shared by its keys already; the published "
                                             "block index applies to the block-addressed file set only"))
        if self.distributed_node_id >= 0:
            out.append(("distributed_node_id", "node ids are allocated by the registry"))
        if (self.local_zmq_ip, self.local_zmq_port) != ("127.0.0.1", 5555):
            out.append(("local_zmq_ip / local_zmq_port", "peers are read through their pool and block files, not "
                                                         "through a per-node ZeroMQ endpoint"))
        return out


def _env(name: str, default: Any, cast=None) -> Any:
    v = os.getenv(name)
    if v is None:
        return default
    if cast is bool:
        return bool(int(v))
    return (cast or type(default))(v)


def assert_mooncake_prefetch_ready(cache_config, prefetch_enabled: bool) -> None:
    """With a key-addressed remote store, compute-path gets stay on the local tiers; the store is read by
    prefetches only. A connector whose prefetch hook is off would never read the store: refuse that
    combination at start-up (reference: flexkv/common/config.py:17-29)."""
    if getattr(cache_config, "use_mooncake_store_backend", False) and not prefetch_enabled \
            and os.environ.get("FLEXKV_REMOTE_STORE_IN_GRAPH", "0") != "1":
        raise RuntimeError("use_mooncake_store_backend needs the connector's prefetch: the store is read ahead of "
                           "scheduling, never on the compute path (or set FLEXKV_REMOTE_STORE_IN_GRAPH=1)")


def load_env_config() -> Namespace:
    return Namespace(
        instance_num=_env("FLEXKV_INSTANCE_NUM", 1),
        instance_id=_env("FLEXKV_INSTANCE_ID", 0),
        enable_metrics=_env("FLEXKV_ENABLE_METRICS", False, bool),
        cpp_metrics_port=_env("FLEXKV_CPP_METRICS_PORT", 8081),
        py_metrics_port=_env("FLEXKV_PY_METRICS_PORT", 8080),
        server_client_mode=_env("FLEXKV_SERVER_CLIENT_MODE", False, bool),
        server_launch_mode=_env("FLEXKV_SERVER_LAUNCH_MODE", "embedded").lower(),
        server_recv_port=_env("FLEXKV_SERVER_RECV_PORT", "ipc:///tmp/flexkv_server"),
        index_accel=_env("FLEXKV_INDEX_ACCEL", True, bool),
        native_scheduler=_env("FLEXKV_NATIVE_SCHEDULER", True, bool),
        # "thread": the data plane shares the serving process (default); "process": it runs in a child process
        transfer_manager_mode=_env("FLEXKV_TRANSFER_MANAGER_MODE", "thread", str),
        crash_diagnostics=_env("FLEXKV_CRASH_DIAGNOSTICS", False, bool),
        cpu_layout_type=KVCacheLayoutType(_env("FLEXKV_CPU_LAYOUT", "BLOCKFIRST").upper()),
        ssd_layout_type=KVCacheLayoutType(_env("FLEXKV_SSD_LAYOUT", "BLOCKFIRST").upper()),
        remote_layout_type=KVCacheLayoutType(_env("FLEXKV_REMOTE_LAYOUT", "BLOCKFIRST").upper()),
        gds_layout_type=KVCacheLayoutType(_env("FLEXKV_GDS_LAYOUT", "BLOCKFIRST").upper()),
        enable_layerwise_transfer=_env("FLEXKV_ENABLE_LAYERWISE_TRANSFER", False, bool),
        # copy kernel launch shape: four single-warp CTAs with 16 KiB tiles already fill a PCIe Gen5 x16 link
        transfer_num_cta_h2d=_env("FLEXKV_TRANSFER_NUM_CTA_H2D", 8),
        transfer_num_cta_d2h=_env("FLEXKV_TRANSFER_NUM_CTA_D2H", 8),
        transfer_tile_bytes=_env("FLEXKV_TRANSFER_TILE_BYTES", 16384),
        transfer_engine=_env("FLEXKV_TRANSFER_ENGINE", "auto").lower(),  # tma | simt | ce | auto
        # copy-engine router: the two switches turn on "auto" per direction; the segment
        # threshold is accepted for compatibility (routing here is by bytes per driver call)
        use_ce_transfer_h2d=_env("FLEXKV_USE_CE_TRANSFER_H2D", False, bool),
        use_ce_transfer_d2h=_env("FLEXKV_USE_CE_TRANSFER_D2H", False, bool),
        ce_segment_threshold=_env("FLEXKV_CE_SEGMENT_THRESHOLD", 8),
        ssd_io_opt=_env("FLEXKV_SSD_IO_OPT", True, bool),
        ssd_io_threads=_env("FLEXKV_SSD_IO_THREADS", 8),
        iouring_entries=_env("FLEXKV_IOURING_ENTRIES", 512),
        iouring_flags=_env("FLEXKV_IOURING_FLAGS", 0),
        max_file_size_gb=_env("FLEXKV_MAX_FILE_SIZE_GB", -1.0),
        ssd_persist=_env("FLEXKV_SSD_PERSIST", False, bool),
        evict_ratio=_env("FLEXKV_EVICT_RATIO", 0.0),
        evict_start_threshold=_env("FLEXKV_EVICT_START_THRESHOLD", 1.0),
        hit_reward_seconds=_env("FLEXKV_HIT_REWARD_SECONDS", 0),
        eviction_policy=_env("FLEXKV_EVICTION_POLICY", "lru"),
        slru_protected_threshold=_env("FLEXKV_SLRU_PROTECTED_THRESHOLD", 2),
        enable_mps=_env("FLEXKV_ENABLE_MPS", False, bool),
        enable_collective_sync=_env("FLEXKV_ENABLE_COLLECTIVE_SYNC", True, bool),
        enable_trace=_env("FLEXKV_ENABLE_TRACE", False, bool),
        trace_file_path=_env("FLEXKV_TRACE_FILE_PATH", "./flexkv_trace.log"),
        trace_max_file_size_mb=_env("FLEXKV_TRACE_MAX_FILE_SIZE_MB", 100),
        trace_max_files=_env("FLEXKV_TRACE_MAX_FILES", 5),
        trace_flush_interval_ms=_env("FLEXKV_TRACE_FLUSH_INTERVAL_MS", 1000),
        enable_transfer_trace=_env("FLEXKV_TRANSFER_TRACE", False, bool),
        refresh_batch_size=_env("FLEXKV_REFRESH_BATCH_SIZE", 256),
        rebuild_interval_ms=_env("FLEXKV_REBUILD_INTERVAL_MS", 2000),
        idle_sleep_ms=_env("FLEXKV_IDLE_SLEEP_MS", 10),
        lease_ttl_ms=_env("FLEXKV_LEASE_TTL_MS", 30000),
        safety_ttl_ms=_env("FLEXKV_SAFETY_TTL_MS", 100),
        renew_lease_ms=_env("FLEXKV_RENEW_LEASE_MS", 4000),
        reset_barrier_timeout_ms=_env("FLEXKV_RESET_BARRIER_TIMEOUT_MS", 60000),
        reset_barrier_poll_ms=_env("FLEXKV_RESET_BARRIER_POLL_MS", 50),
        enable_compression=_env("FLEXKV_ENABLE_NVCOMP", False, bool),
        kv_shared_across_ranks_mode=_env("FLEXKV_KV_SHARED_ACROSS_RANKS_MODE", "sharded"),
        layerwise_notify_mode=_env("FLEXKV_LAYERWISE_NOTIFY_MODE", "hostfunc"),
        worker_shutdown_timeout_s=_env("FLEXKV_WORKER_SHUTDOWN_TIMEOUT_S", 600.0),
        transfer_manager_shutdown_timeout_s=_env("FLEXKV_TRANSFER_MANAGER_SHUTDOWN_TIMEOUT_S", 900.0),
        log_level=_env("FLEXKV_LOG_LEVEL", "INFO"),
        task_ttl_seconds=_env("FLEXKV_TASK_TTL_SECONDS", 1800),
    )


GLOBAL_CONFIG_FROM_ENV: Namespace = load_env_config()


@dataclass
class UserConfig:
    """What a deployment sets: sizes in GB, directories and feature switches
    (file at ``FLEXKV_CONFIG_PATH`` as json or yaml, or ``FLEXKV_*`` variables)."""
    cpu_cache_gb: float = 16
    ssd_cache_gb: float = 0
    ssd_cache_dir: Union[str, List[str]] = "/data/flexkv_ssd/"
    enable_gds: bool = False
    use_hugepage_cpu_buffer: bool = False
    use_hugepage_tmp_buffer: bool = False
    hugepage_size_bytes: int = 2 * 1024 * 1024
    enable_p2p_cpu: bool = False
    enable_p2p_ssd: bool = False
    enable_p2p_gpu: bool = False
    redis_host: str = "127.0.0.1"
    redis_port: int = 6379
    redis_password: Optional[str] = None
    local_ip: str = "127.0.0.1"
    kv_cache_dtype: Optional[str] = None
    offload_quant: str = "none"
    # keys a deployment file written for the reference may carry (flexkv/common/config.py:843-880); they are
    # passed on to CacheConfig, which reports the ones that have no effect in this build
    enable_nixl: bool = False
    enable_3rd_remote: bool = False
    use_mooncake_store_backend: bool = False
    mooncake_store_config_path: Optional[str] = None
    mooncake_store_pp_rank: int = 0
    mooncake_store_pp_size: int = 1
    mooncake_store_node_layer_start: int = 0
    mooncake_store_node_layer_end: int = 0
    mooncake_store_total_layers: int = 0
    local_zmq_ip: Optional[str] = None
    local_zmq_port: Optional[int] = None
    node_ttl_seconds: Optional[int] = None
    swa_multi_group: Optional[bool] = None
    overrides: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.cpu_cache_gb <= 0:
            raise ValueError("cpu_cache_gb must be positive")
        if self.ssd_cache_gb < 0:
            raise ValueError("ssd_cache_gb must be non-negative")
        if 0 < self.ssd_cache_gb <= self.cpu_cache_gb:
            raise ValueError("ssd_cache_gb must exceed cpu_cache_gb when the SSD tier is on")


def parse_path_list(path_str: Union[str, List[str]]) -> List[str]:
    if isinstance(path_str, (list, tuple)):
        return [str(p) for p in path_str]
    return [p.strip() for p in str(path_str).split(";") if p.strip()]


def _coerce(value: Any, like: Any) -> Any:
    if isinstance(like, bool):
        if isinstance(value, str):
            return value.strip().lower() in ("1", "true", "yes", "on")
        return bool(value)
    if isinstance(like, KVCacheLayoutType):
        return KVCacheLayoutType(str(value).upper())
    if isinstance(like, int) and not isinstance(like, bool):
        try:
            return int(value)
        except ValueError:
            f = float(value)              # sizes in GB may be fractional ("0.5"); anything else raises here
            return int(f) if f.is_integer() else f
    if isinstance(like, float):
        return float(value)
    return value


def load_user_config_from_file(path: str) -> UserConfig:
    with open(path) as f:
        if path.endswith((".yaml", ".yml")):
            import yaml
            raw = yaml.safe_load(f) or {}
        else:
            raw = json.load(f)
    known = {f.name for f in fields(UserConfig)}
    kw = {k: v for k, v in raw.items() if k in known and k != "overrides"}
    cfg = UserConfig(**kw)
    # anything else addresses the environment table by its attribute name
    cfg.overrides = {k: v for k, v in raw.items() if k not in known}
    return cfg


def load_user_config_from_env() -> UserConfig:
    path = os.getenv("FLEXKV_CONFIG_PATH")
    if path:
        return load_user_config_from_file(path)
    kw: Dict[str, Any] = {}
    for f in fields(UserConfig):
        if f.name == "overrides":
            continue
        v = os.getenv("FLEXKV_" + f.name.upper())
        if v is not None:
            kw[f.name] = _coerce(v, f.default) if f.default is not None else v
    return UserConfig(**kw)


def apply_overrides(user: UserConfig, env: Optional[Namespace] = None) -> None:
    env = env if env is not None else GLOBAL_CONFIG_FROM_ENV
    for k, v in user.overrides.items():
        key = k[len("override_"):] if k.startswith("override_") else k
        if not hasattr(env, key):
            raise ValueError(f"unknown config key: {k}")
        setattr(env, key, _coerce(v, getattr(env, key)))


def convert_to_block_num(size_in_gb: float, block_size_in_bytes: int) -> int:
    return int(size_in_gb * (1 << 30)) // max(1, block_size_in_bytes)


def update_default_config_from_user_config(model_config: ModelConfig, cache_config: CacheConfig,
                                           user_config: UserConfig) -> None:
    """Fills block counts and tier switches of ``cache_config`` from sizes in GB."""
    if user_config.kv_cache_dtype and not model_config._frozen:
        model_config.dtype = parse_dtype(user_config.kv_cache_dtype)
    block_bytes = model_config.block_size_in_bytes(cache_config.tokens_per_block)
    if cache_config.offload_quant == "none" and user_config.offload_quant != "none":
        cache_config.offload_quant = user_config.offload_quant
    cache_config._user_cpu_cache_gb = user_config.cpu_cache_gb
    cache_config._user_ssd_cache_gb = user_config.ssd_cache_gb
    cache_config.num_cpu_blocks = convert_to_block_num(user_config.cpu_cache_gb, block_bytes)
    cache_config.enable_cpu = True
    cache_config.use_hugepage_cpu_buffer = user_config.use_hugepage_cpu_buffer
    cache_config.use_hugepage_tmp_buffer = user_config.use_hugepage_tmp_buffer
    cache_config.hugepage_size_bytes = user_config.hugepage_size_bytes
    if user_config.ssd_cache_gb > 0:
        dirs = parse_path_list(user_config.ssd_cache_dir)
        cache_config.enable_ssd = True
        cache_config.ssd_cache_dir = dirs
        n = convert_to_block_num(user_config.ssd_cache_gb, block_bytes)
        cache_config.num_ssd_blocks = n - n % max(1, len(dirs))
        cache_config.enable_gds = user_config.enable_gds
    else:
        cache_config.enable_ssd = False
        cache_config.num_ssd_blocks = 0
    cache_config.enable_p2p_cpu = user_config.enable_p2p_cpu
    cache_config.enable_p2p_ssd = user_config.enable_p2p_ssd
    cache_config.enable_p2p_gpu = user_config.enable_p2p_gpu
    cache_config.redis_host = user_config.redis_host
    cache_config.redis_port = user_config.redis_port
    cache_config.redis_password = user_config.redis_password
    cache_config.local_ip = user_config.local_ip
    cache_config.enable_nixl = bool(user_config.enable_nixl)
    cache_config.enable_3rd_remote = bool(user_config.enable_3rd_remote)
    cache_config.use_mooncake_store_backend = bool(user_config.use_mooncake_store_backend)
    if user_config.mooncake_store_config_path:
        cache_config.mooncake_store_config_path = user_config.mooncake_store_config_path
    if user_config.local_zmq_ip:
        cache_config.local_zmq_ip = user_config.local_zmq_ip
    if user_config.local_zmq_port:
        cache_config.local_zmq_port = int(user_config.local_zmq_port)
    if user_config.node_ttl_seconds:
        cache_config.node_ttl_seconds = int(user_config.node_ttl_seconds)
    # None / True: compressor-state sidecars travel with the window slot; False keeps the window-only path. The
    # engine adapter that reads the pool (SGLang) takes the switch from here.
    cache_config._swa_multi_group = user_config.swa_multi_group
    if user_config.swa_multi_group is False and cache_config.swa is not None:
        cache_config.swa.sidecar_groups = []
    cache_config.__post_init__()
    apply_overrides(user_config)


def recompute_block_counts(model_config: ModelConfig, cache_config: CacheConfig) -> None:
    """Called when layer groups become known after the first sizing."""
    block_bytes = model_config.block_size_in_bytes(cache_config.tokens_per_block)
    if cache_config._user_cpu_cache_gb:
        cache_config.num_cpu_blocks = convert_to_block_num(cache_config._user_cpu_cache_gb, block_bytes)
    if cache_config._user_ssd_cache_gb and cache_config.enable_ssd:
        dirs = parse_path_list(cache_config.ssd_cache_dir or [])
        n = convert_to_block_num(cache_config._user_ssd_cache_gb, block_bytes)
        cache_config.num_ssd_blocks = n - n % max(1, len(dirs))
