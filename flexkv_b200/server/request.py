"""Messages between clients and the KV server (flexkv/server/request.py:15-180)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np

from ..common.memory_handle import TensorSharedHandle
from ..common.storage import KVCacheLayout


@dataclass
class Request:
    dp_client_id: int = 0
    seq: int = 0                      # echoed in the response so a client can pair them


@dataclass
class RegisterDPClientRequest(Request):
    client_recv_port: str = ""


@dataclass
class RegisterTPClientRequest:
    """One engine worker's KV tensors; key = (dp_client_id, intra_client_id)
    (flexkv/server/request.py:46-48)."""
    dp_client_id: int
    intra_client_id: int              # pp_rank * effective_tp + effective_tp_rank
    device_id: int
    handles: List[TensorSharedHandle]
    gpu_layout: KVCacheLayout
    pp_rank: int = 0
    tp_rank: int = 0
    group_id: int = -1               # layer group of a multi-group cache (window pages: group of the window pool)
    is_swa: bool = False             # the tensors are sliding-window pages ([pages, page bytes] per layer)
    layer_groups: Optional[List[Any]] = None   # LayerGroupSpec list when the worker discovered the groups itself


@dataclass
class SlotMappingRequest:
    """The GPU pages one node's ranks allocated for a task whose graph arrives from the master node with its GPU
    side unbound: each node of a group that spans nodes has its own block numbering
    (flexkv/server/client.py:308-334 ``set_slot_mapping``, flexkv/kvtask.py:438-444)."""
    task_id: int
    slot_mapping: Any                  # int64 numpy array, one slot per token
    dp_client_id: int = 0


@dataclass
class GpuControlRequest:
    """Sleep / wake of one engine worker's GPU memory, sent on the registration channel
    (the reference uses a dedicated REP socket: flexkv/transfer_manager.py:167-245).
    ``registration`` carries the handles of the re-created tensors on resume."""
    dp_client_id: int
    action: str                        # "suspend" | "resume"
    reply_endpoint: str = ""
    registration: Optional[RegisterTPClientRequest] = None
    timeout: float = 60.0
    more_registrations: Optional[List[RegisterTPClientRequest]] = None    # the other groups of a multi-group cache


@dataclass
class IsReadyRequest(Request):
    pass


@dataclass
class PutRequest(Request):
    token_ids: np.ndarray = None
    slot_mapping: Optional[np.ndarray] = None
    token_mask: Optional[np.ndarray] = None
    namespace: Optional[List[str]] = None
    match_only: bool = False


@dataclass
class GetRequest(Request):
    token_ids: np.ndarray = None
    slot_mapping: Optional[np.ndarray] = None
    token_mask: Optional[np.ndarray] = None
    namespace: Optional[List[str]] = None
    match_only: bool = False
    cpu_only: bool = False
    swa_aware: bool = False


@dataclass
class PrefetchRequest(Request):
    token_ids: np.ndarray = None
    namespace: Optional[List[str]] = None
    swa_aware: bool = False


@dataclass
class LaunchRequest(Request):
    task_ids: List[int] = field(default_factory=list)
    slot_mappings: List[np.ndarray] = field(default_factory=list)
    as_batch: bool = False
    layerwise_transfer: bool = False
    counter_id: int = 0


@dataclass
class CancelRequest(Request):
    task_ids: List[int] = field(default_factory=list)


@dataclass
class WaitRequest(Request):
    task_ids: List[int] = field(default_factory=list)
    timeout: float = 20.0
    completely: bool = False
    try_wait: bool = False


@dataclass
class ResetRequest(Request):
    pass


@dataclass
class PublishGpuBlocksRequest(Request):
    token_ids: np.ndarray = None
    slot_mapping: np.ndarray = None
    namespace: Optional[List[str]] = None


@dataclass
class WithdrawGpuBlocksRequest(Request):
    gpu_block_ids: np.ndarray = None


@dataclass
class ShutdownRequest(Request):
    pass


@dataclass
class UnregisterDPClientRequest(Request):
    """One data-parallel client leaves; the shared server keeps running for the others
    (flexkv/server/server.py:486-490)."""


@dataclass
class Response:
    dp_client_id: int
    seq: int = 0
    task_id: Optional[int] = None
    task_ids: Optional[List[int]] = None
    mask: Optional[np.ndarray] = None
    status: Optional[Dict[int, Any]] = None
    ready: Optional[bool] = None
    value: Any = None
    error: Optional[str] = None
