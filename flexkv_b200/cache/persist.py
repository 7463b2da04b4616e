"""Warm restart of the SSD tier: the prefix index of a tier whose bytes outlive the
process is written beside the cache files at shutdown and mounted again at start.

The reference keeps its SSD index in memory only, so every restart begins cold
(flexkv/cache/cache_engine.py:1-120 builds empty trees; flexkv/storage/allocator.py
recreates the files). Here a clean shutdown leaves three things in the first cache
directory:

* ``flexkv_ssd_cache_<dev>_<n>.bin``  the block files (fixed names, not removed),
* ``flexkv_ssd_cache.index.npz``      the ready part of the index (native pre-order image)
                                      plus a signature of everything that decides where a
                                      block's bytes are and what they mean,
* ``flexkv_ssd_cache.sizes.npy``      the per-tile size table of the lossless codec (an empty
                                      array otherwise), written by the data plane before the
                                      index, whose signature carries its size, mtime and shape.

The index file is consumed by the load (renamed to ``.mounted``): it only ever describes the
files as a clean shutdown left them, so a crash after the mount cannot bring back an index
that is older than the bytes on disk.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import numpy as np

from ..common.config import GLOBAL_CONFIG_FROM_ENV, CacheConfig, ModelConfig, parse_path_list
from ..common.debug import flexkv_logger

FORMAT = "flexkv_b200.ssd_index.v1"
FILE_PREFIX = "flexkv_ssd_cache"


def persist_enabled(cache_config: CacheConfig) -> bool:
    return bool(cache_config.enable_ssd and
                (getattr(cache_config, "ssd_persist", False) or GLOBAL_CONFIG_FROM_ENV.ssd_persist))


def _first_dir(cache_config: CacheConfig) -> str:
    dirs = parse_path_list(cache_config.ssd_cache_dir or [])
    if not dirs:
        raise ValueError("enable_ssd requires ssd_cache_dir")
    return dirs[0]


def index_path(cache_config: CacheConfig) -> str:
    return os.path.join(_first_dir(cache_config), FILE_PREFIX + ".index.npz")


def size_table_path(cache_config: CacheConfig) -> str:
    return os.path.join(_first_dir(cache_config), FILE_PREFIX + ".sizes.npy")


def signature(cache_config: CacheConfig, model_config: ModelConfig) -> Dict[str, Any]:
    """Everything that fixes the meaning of SSD block ``i``: geometry of one block, the block
    count and its striping over directories, the host codec, and the key function's inputs."""
    m, c = model_config, cache_config
    env = GLOBAL_CONFIG_FROM_ENV
    return {
        "format": FORMAT,
        "tokens_per_block": int(c.tokens_per_block),
        "num_ssd_blocks": int(c.num_ssd_blocks),
        "ssd_dirs": len(parse_path_list(c.ssd_cache_dir or [])),
        "max_file_size_gb": float(env.max_file_size_gb),
        "num_layers": int(m.num_layers),
        "num_kv_heads": int(m.num_kv_heads),
        "head_size": int(m.head_size),
        "use_mla": bool(m.use_mla),
        "dtype": str(m.dtype),
        "tp_size": int(m.tp_size),
        "pp_size": int(getattr(m, "pp_size", 1)),
        "local_pp_stages": int(getattr(m, "local_pp_stages", 1)),
        "offload_quant": str(c.offload_quant),
        # inputs of the host codec decision (the codec fixes the bytes of a block)
        "compression": bool(c.enable_compression or env.enable_compression),
        "codec_format": 2,      # layout of a packed tile (rank-coded exponents); bump when the bytes change
        "layerwise": bool(env.enable_layerwise_transfer),
        "p2p_cpu": bool(c.enable_p2p_cpu),
        "host_layout": str(env.cpu_layout_type),
        "ssd_layout": str(env.ssd_layout_type),
    }


def save_size_table(cache_config: CacheConfig, table: Optional[np.ndarray]) -> None:
    """The data plane's half of a clean shutdown: the per-tile size table of the SSD blocks
    (an empty array when the tier holds raw or fixed-size blocks). Written before the index."""
    path = size_table_path(cache_config)
    tmp = path + f".tmp{os.getpid()}"
    try:
        with open(tmp, "wb") as f:
            np.save(f, table if table is not None else np.zeros((0,), dtype=np.int32))
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except OSError as e:
        flexkv_logger.warning("ssd size table not saved (%s): %s", path, e)


def load_size_table(cache_config: CacheConfig, table: Optional[np.ndarray]) -> bool:
    """Fills ``table`` from the saved one when the shapes agree. The file stays in place:
    only the index decides whether the saved state is used."""
    path = size_table_path(cache_config)
    if table is None or not os.path.exists(path):
        return False
    try:
        saved = np.load(path, mmap_mode="r")
        if saved.shape != table.shape or saved.dtype != table.dtype:
            return False
        table[...] = saved
        return True
    except Exception as e:  # noqa: BLE001
        flexkv_logger.warning("ssd size table unreadable (%s): %s", path, e)
        return False


def _table_stamp(cache_config: CacheConfig) -> Optional[list]:
    """Identity of the size-table file the index was saved against."""
    path = size_table_path(cache_config)
    try:
        st = os.stat(path)
        shape = list(np.load(path, mmap_mode="r").shape)
    except Exception:  # noqa: BLE001
        return None
    return [int(st.st_size), int(st.st_mtime_ns), shape]


def save_index(cache_config: CacheConfig, model_config: ModelConfig, engine) -> Optional[str]:
    """Writes the ready part of ``engine``'s index (a ``CacheEngine`` of the SSD tier).
    Atomic: a temporary file in the same directory is renamed over the target."""
    path = index_path(cache_config)
    parents, sizes, hashes, blocks = engine.index.export_ready()
    tmp = path + f".tmp{os.getpid()}"
    try:
        with open(tmp, "wb") as f:
            sig = dict(signature(cache_config, model_config), size_table=_table_stamp(cache_config))
            np.savez(f, signature=np.frombuffer(json.dumps(sig, sort_keys=True).encode(), dtype=np.uint8),
                     parents=parents, sizes=sizes, hashes=hashes, blocks=blocks)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except OSError as e:
        flexkv_logger.warning("ssd index not saved (%s): %s", path, e)
        try:
            os.unlink(tmp)
        except OSError:
            pass
        return None
    flexkv_logger.info("ssd index saved: %d blocks in %d nodes -> %s", len(blocks), len(parents), path)
    return path


def load_index(cache_config: CacheConfig, model_config: ModelConfig, engine) -> int:
    """Mounts a saved index into the (empty) SSD ``engine`` and takes its blocks out of the
    free pool. Returns the number of blocks restored; 0 when there is no usable image (none
    saved, another geometry or codec, a damaged file, a size table that should exist and
    does not). The image is renamed to ``.mounted`` whatever the outcome."""
    path = index_path(cache_config)
    if not os.path.exists(path):
        return 0
    try:
        with np.load(path) as z:
            saved = json.loads(bytes(z["signature"]).decode())
            arrays = (z["parents"], z["sizes"], z["hashes"], z["blocks"])
    except Exception as e:  # noqa: BLE001 - any damaged file means a cold start
        flexkv_logger.warning("ssd index unreadable (%s): %s", path, e)
        _consume(path)
        return 0
    _consume(path)
    want = dict(signature(cache_config, model_config), size_table=_table_stamp(cache_config))
    if saved != want:
        diff = sorted(k for k in set(saved) | set(want) if saved.get(k) != want.get(k))
        flexkv_logger.warning("ssd index ignored, saved state differs in %s", diff)
        return 0
    if want["size_table"] is None:
        flexkv_logger.warning("ssd index ignored, the data plane left no size table beside it")
        return 0
    try:
        n = int(engine.index.import_snapshot(*arrays))
        engine.mempool.reserve_blocks(arrays[3])
    except (ValueError, RuntimeError, IndexError) as e:
        flexkv_logger.warning("ssd index ignored, image rejected: %s", e)
        engine.reset()
        return 0
    flexkv_logger.info("ssd index mounted: %d blocks in %d nodes from %s", n, len(arrays[0]), path)
    return n


def discard_index(cache_config: CacheConfig) -> None:
    """Removes a saved image that no longer describes the files (blocks are about to be rewritten)."""
    try:
        os.unlink(index_path(cache_config))
    except OSError:
        pass


def _consume(path: str) -> None:
    try:
        os.replace(path, path + ".mounted")
    except OSError:
        pass
