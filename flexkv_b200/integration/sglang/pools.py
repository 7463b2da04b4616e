"""What an SGLang KV pool object consists of, as layer groups and window pools.

The connector never imports SGLang; it reads the pool object's attributes:

* plain pools: ``kv_buffer`` (MLA, one tensor per layer) or ``k_buffer`` / ``v_buffer``; an optional
  ``index_k_with_scale_buffer`` (indexer keys beside every layer) becomes a second layer group;
* split compressed-attention pools (DeepSeek-V4 style): ``compression_ratios`` per model layer,
  ``c4_kv_pool`` / ``c128_kv_pool`` (``kv_buffer``, ``page_size``, ``get_bytes_per_token()``),
  ``c4_indexer_kv_pool.index_k_with_scale_buffer``, a sliding-window pool (``swa_kv_pool.kv_buffer``)
  and, per compressed layer, compressor state pools (``compress_state_pools`` /
  ``indexer_compress_state_pools`` with ``ring_size`` and ``kv_score_buffer.kv_score``) that ride in
  the window slot as sidecar groups

(reference behaviour: flexkv/integration/sglang/connector.py:1599-1807 ``_resolve_kv_buffers``,
``_append_dsv4_state_group``, ``_build_dsv4_layer_group_specs``, ``_build_indexer_layer_group_specs``;
:1876-1897 ``_build_swa_slot_mapping``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch

from ...common.config import LayerGroupSpec, SWAPoolConfig


@dataclass
class PoolGroup:
    name: str
    ratio: int                      # tokens of the model per stored token
    layer_ids: List[int]            # model layers (local to this pipeline stage) the buffers belong to
    buffers: List[torch.Tensor]     # one per layer, viewable as [pages, page bytes]
    sub_page_size: int              # stored tokens per page
    bytes_per_token: int
    dtype: torch.dtype = torch.uint8


@dataclass
class ResolvedPool:
    kind: str                                   # "mha" | "mla" | "indexer" | "split"
    groups: List[PoolGroup] = field(default_factory=list)
    k_buffers: List[torch.Tensor] = field(default_factory=list)     # plain pools
    v_buffers: Optional[List[torch.Tensor]] = None
    swa_buffers: List[torch.Tensor] = field(default_factory=list)   # window KV, one tensor per window layer
    state_groups: List[PoolGroup] = field(default_factory=list)     # sidecars of the window slot

    @property
    def multi_group(self) -> bool:
        return self.kind in ("split", "indexer")


def _pages(buf: torch.Tensor, num_pages: int) -> torch.Tensor:
    """``buf`` as [pages, page bytes] (uint8), without copying."""
    flat = buf.reshape(-1).view(torch.uint8) if buf.is_contiguous() else None
    if flat is None or flat.numel() % num_pages:
        raise RuntimeError(f"buffer of shape {tuple(buf.shape)} cannot be split into {num_pages} contiguous pages")
    return flat.view(num_pages, flat.numel() // num_pages)


def resolve_kv_pool(kvcache: Any, page_size: int, include_state: Optional[bool] = None) -> ResolvedPool:
    indexer = list(getattr(kvcache, "index_k_with_scale_buffer", None) or [])
    if not hasattr(kvcache, "compression_ratios"):
        if hasattr(kvcache, "kv_buffer"):
            out = ResolvedPool("mla", k_buffers=list(kvcache.kv_buffer))
        elif hasattr(kvcache, "k_buffer"):
            out = ResolvedPool("mha", k_buffers=list(kvcache.k_buffer), v_buffers=list(kvcache.v_buffer))
        else:
            raise AttributeError(f"unsupported KV pool {type(kvcache).__name__}: expected kv_buffer, "
                                 "k_buffer/v_buffer or split compressed pools")
        if indexer:
            # indexer keys beside every layer: a second, byte-wise layer group
            num_pages = out.k_buffers[0].shape[0] // page_size
            pages = [_pages(b, num_pages) for b in indexer]
            out.groups = [PoolGroup("indexer", 1, list(range(len(indexer))), pages, page_size,
                                    pages[0].shape[1] // page_size)]
            out.kind = "indexer"
        return out

    if getattr(kvcache, "_unified_kv", False):
        raise NotImplementedError("the split c4 / c128 / window layout is required; a unified KV pool is not supported")
    ratios = list(kvcache.compression_ratios)
    lo = int(getattr(kvcache, "_stage_start", 0))
    hi = int(getattr(kvcache, "_stage_end", len(ratios)))
    out = ResolvedPool("split")

    def add(name: str, ratio: int, layer_ids: List[int], buffers, sub_page: int, bpt: int) -> None:
        buffers = list(buffers or [])
        if not buffers:
            return
        if len(buffers) != len(layer_ids):
            raise RuntimeError(f"pool group {name!r}: {len(buffers)} buffers for {len(layer_ids)} layers")
        pages = [b if b.ndim == 2 else b.reshape(b.shape[0], -1) for b in buffers]
        if pages[0].shape[1] * pages[0].element_size() % int(sub_page):
            raise RuntimeError(f"pool group {name!r}: page of {pages[0].shape[1]} elements is not a whole number "
                               f"of {sub_page} stored tokens")
        out.groups.append(PoolGroup(name, ratio, layer_ids, pages, int(sub_page), int(bpt), pages[0].dtype))

    c4_global = [i for i in range(lo, hi) if ratios[i] == 4]
    c128_global = [i for i in range(lo, hi) if ratios[i] == 128]
    c4, c128 = [i - lo for i in c4_global], [i - lo for i in c128_global]
    p4, p128 = getattr(kvcache, "c4_kv_pool", None), getattr(kvcache, "c128_kv_pool", None)
    if p4 is not None:
        add("c4", 4, c4, p4.kv_buffer, p4.page_size, p4.get_bytes_per_token())
    if p128 is not None:
        add("c128", 128, c128, p128.kv_buffer, p128.page_size, p128.get_bytes_per_token())
    pidx = getattr(kvcache, "c4_indexer_kv_pool", None)
    idx_bufs = list(getattr(pidx, "index_k_with_scale_buffer", []) or []) if pidx is not None else []
    if idx_bufs:
        add("c4_indexer", 4, list(c4), idx_bufs, pidx.page_size, idx_bufs[0].shape[1] // pidx.page_size)
    if not out.groups:
        raise RuntimeError("the split KV pool has no buffers on this pipeline stage")

    swa_pool = getattr(kvcache, "swa_kv_pool", None)
    if swa_pool is not None:
        out.swa_buffers = [b if b.ndim == 2 else b.reshape(b.shape[0], -1) for b in swa_pool.kv_buffer]
    if include_state is not False and out.swa_buffers:
        swa_page = int(getattr(kvcache, "swa_page_size", page_size))
        for name, attr in (("c4_attention_state", "compress_state_pools"),
                           ("c4_indexer_state", "indexer_compress_state_pools")):
            pools = [getattr(kvcache, attr)[i] for i in c4_global] if hasattr(kvcache, attr) else []
            if not pools or any(p is None for p in pools):
                continue
            rings = {int(p.ring_size) for p in pools}
            if len(rings) != 1:
                raise RuntimeError(f"state group {name!r} has mixed ring sizes {sorted(rings)}")
            ring = rings.pop()
            if swa_page != page_size or swa_page % ring:
                raise RuntimeError(f"state group {name!r}: page size {swa_page} and ring size {ring} do not fit")
            bufs = [p.kv_score_buffer.kv_score for p in pools]
            s0 = bufs[0]
            if s0.ndim != 2 or any(b.shape != s0.shape or b.dtype != s0.dtype or not b.is_contiguous() for b in bufs):
                raise RuntimeError(f"state group {name!r} expects identical contiguous 2-D buffers")
            num_pages = s0.shape[0] // ring
            out.state_groups.append(PoolGroup(name, swa_page // ring, list(c4), [_pages(b, num_pages) for b in bufs],
                                              ring, s0.shape[1] * s0.element_size(), s0.dtype))
    return out


def layer_group_specs(pool: ResolvedPool, page_size: int) -> Optional[List[LayerGroupSpec]]:
    """The ``ModelConfig.layer_groups`` this pool needs (None for a plain single-group cache). Every group is
    described byte-wise: one "head" of ``bytes per stored token`` uint8 values, ``page_size / ratio`` tokens a block."""
    if not pool.multi_group:
        return None
    specs = []
    if pool.kind == "indexer":
        # the main cache keeps its element-wise description: [tokens, heads, head] per layer (K and V, or MLA)
        t = pool.k_buffers[0]
        heads, head = (int(t.shape[-2]), int(t.shape[-1])) if t.ndim >= 3 else (1, int(t.shape[-1]))
        specs.append(LayerGroupSpec(num_layers=len(pool.k_buffers), num_kv_heads=heads, head_size=head,
                                    kv_dim=1 if pool.v_buffers is None else 2, dtype=t.dtype,
                                    layer_ids=list(range(len(pool.k_buffers))), name="kv"))
    for g in pool.groups:
        page_bytes = g.buffers[0].shape[1] * g.buffers[0].element_size()
        specs.append(LayerGroupSpec(num_layers=len(g.layer_ids), num_kv_heads=1, head_size=page_bytes // g.sub_page_size,
                                    kv_dim=1, dtype=torch.uint8, compress_ratio=max(1, page_size // g.sub_page_size),
                                    layer_ids=list(g.layer_ids), name=g.name))
    return specs


def window_pool_config(pool: ResolvedPool, page_size: int, base: Optional[SWAPoolConfig] = None
                       ) -> Optional[SWAPoolConfig]:
    """Fills the geometry of the window pool (and its sidecar groups) from the resolved buffers."""
    if not pool.swa_buffers:
        return base
    cfg = base if base is not None else SWAPoolConfig(enabled=True)
    s0 = pool.swa_buffers[0]
    cfg.enabled = True
    cfg.num_swa_layers = len(pool.swa_buffers)
    cfg.bytes_per_token_per_layer = s0.shape[1] * s0.element_size() // page_size
    cfg.sidecar_groups = [(len(g.buffers), g.buffers[0].shape[1] * g.buffers[0].element_size())
                          for g in pool.state_groups]
    cfg.multi_group = bool(pool.state_groups)
    cfg.wait_for_registration = True
    return cfg


def build_swa_slot_mapping(kvcache: Any, full_indices: torch.Tensor) -> Optional[torch.Tensor]:
    """Window-pool slots of a request's tokens: the full-pool indices are translated by the pool and only the
    mapped tail is kept (tokens that already slid out of the window map to the reserved slot 0)."""
    translate = getattr(kvcache, "translate_loc_from_full_to_swa", None)
    if translate is None or getattr(kvcache, "swa_kv_pool", None) is None:
        return None
    swa = translate(full_indices).to(device="cpu", dtype=torch.int64)
    mapped = swa > 0
    if not bool(mapped.any()):
        return None
    holes = (~mapped).nonzero(as_tuple=False)
    if holes.numel():
        swa = swa[int(holes[-1].item()) + 1:]
    if swa.numel() == 0:
        return None
    if not bool((swa > 0).all()):
        raise RuntimeError("the window slot mapping contains the reserved slot 0")
    return swa
