"""Request / response types of the public API. Names and wire values are the reference's
(flexkv/common/request.py:9-42), so engine adapters written against it keep working; the
helpers on ``KVResponse`` are additions."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

Mask = Union[np.ndarray, List[np.ndarray]]


class KVResponseStatus(enum.Enum):
    """Outcome of ``wait`` / ``try_wait`` for one task."""
    SUCCESS = "success"          # the bytes named by the return mask have landed
    FAILED = "failed"            # a transfer op failed; nothing of the task may be relied on
    CANCELLED = "cancelled"      # cancelled before launch, reservations returned
    TIMEOUT = "timeout"          # still running when the caller's time ran out
    UNREADY = "unready"          # matched but not launched yet (no slot mapping bound)
    NOTFOUND = "not_found"       # unknown id, or the answer was already fetched

    @property
    def terminal(self) -> bool:
        return self in (KVResponseStatus.SUCCESS, KVResponseStatus.FAILED, KVResponseStatus.CANCELLED,
                        KVResponseStatus.NOTFOUND)


class KVRequestType(enum.Enum):
    PUT = "put"
    GET = "get"
    PREFETCH = "prefetch"
    SHUTDOWN = "shutdown"


@dataclass
class KVResponse:
    status: KVResponseStatus
    task_id: int
    # per-token mask of what was served / stored; a batch task carries one mask per member
    return_mask: Optional[Mask]

    @property
    def ok(self) -> bool:
        return self.status is KVResponseStatus.SUCCESS

    def num_tokens(self) -> int:
        """Tokens covered by the mask(s)."""
        if self.return_mask is None:
            return 0
        masks: Sequence[np.ndarray] = self.return_mask if isinstance(self.return_mask, list) else [self.return_mask]
        return int(sum(int(np.count_nonzero(m)) for m in masks))

    def get_mask(self, idx: int) -> torch.Tensor:
        """Mask of member ``idx`` of a batch task, as a torch tensor."""
        if not isinstance(self.return_mask, list):
            raise AssertionError("return_mask is not a list of masks")
        if not 0 <= idx < len(self.return_mask):
            raise AssertionError(f"member {idx} out of range ({len(self.return_mask)} masks)")
        return torch.from_numpy(self.return_mask[idx])


@dataclass
class KVRequest:
    """One queued API call (used by the tracer and the replay tool)."""
    request_type: KVRequestType
    request_id: int
    token_ids: np.ndarray
    token_mask: Optional[np.ndarray] = None
    slot_mapping: Optional[np.ndarray] = None
    layer_granularity: int = -1
    dp_id: int = 0
    namespace: Optional[List[str]] = field(default=None)
