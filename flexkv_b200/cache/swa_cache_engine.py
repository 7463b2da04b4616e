"""Sliding-window side ops of a transfer plan.

Window snapshots are mounted on the radix nodes of the host tier; the planner resolves
which slot feeds a get and which slot a put fills. This module only appends the matching
side ops to the plan's graph: standard transfer types flagged ``is_swa=True`` whose block
ids are window-pool slot ids on the host side and window page ids on the GPU side, so the
transfer engine routes them to the window worker (reference:
flexkv/cache/swa_cache_engine.py:142-239 ``build_get_chain`` / ``build_put_chain``).
The host tier and, with ``SWAPoolConfig.num_ssd_slots`` / ``num_remote_slots``, the SSD tier and the
block-addressed remote tier carry snapshots: a put writes the page through host slot -> tier slot, a
get whose deepest snapshot sits on a deeper tier stages it through a temporary host slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from ..common.transfer import DeviceType, TransferOp, TransferOpGraph, TransferType

_EMPTY = np.zeros(0, dtype=np.int64)


@dataclass
class SWAPutChainOpIds:
    d2h_id: Optional[int] = None


class SWAOpConstructor:
    def __init__(self, global_cache_engine) -> None:
        self._gce = global_cache_engine

    @property
    def enabled(self) -> bool:
        cfg = self._gce.cache_config
        eng = self._gce.cache_engines.get(DeviceType.CPU)
        return bool(cfg.enable_swa_transfer) and eng is not None and eng.swa_enabled

    def build_swa_op(self, graph: TransferOpGraph, transfer_type: TransferType, src_slot_ids, dst_slot_ids,
                     dp_client_id: int = 0, gpu_side: Optional[str] = None) -> Optional[TransferOp]:
        """One side op. ``gpu_side`` names the side bound at launch from the caller's window
        page ("src" for puts, "dst" for gets); the other side holds pool slot ids."""
        if not self.enabled:
            return None
        src = _EMPTY if gpu_side == "src" else np.asarray(src_slot_ids, dtype=np.int64)
        dst = _EMPTY if gpu_side == "dst" else np.asarray(dst_slot_ids, dtype=np.int64)
        if (gpu_side != "src" and src.size == 0) or (gpu_side != "dst" and dst.size == 0):
            return None
        op = TransferOp(graph.graph_id, transfer_type, src, dst, dp_client_id=dp_client_id, is_swa=True,
                        gpu_side=gpu_side)
        graph.add_transfer_op(op)
        return op

    def build_get_chain(self, graph: TransferOpGraph, host_slot: int, dp_client_id: int = 0) -> Optional[TransferOp]:
        """host slot -> GPU window page; the terminal op of the chain is reported with the plan."""
        return self.build_swa_op(graph, TransferType.H2D, [host_slot], _EMPTY, dp_client_id, gpu_side="dst")

    def build_put_chain(self, graph: TransferOpGraph, host_slot: int, dp_client_id: int = 0) -> SWAPutChainOpIds:
        op = self.build_swa_op(graph, TransferType.D2H, _EMPTY, [host_slot], dp_client_id, gpu_side="src")
        return SWAPutChainOpIds(op.op_id if op is not None else None)
