"""Request / response types of the public API (same names and values as the
reference: flexkv/common/request.py:9-42)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Union

import numpy as np
import torch


class KVRequestType(Enum):
    GET = "get"
    PUT = "put"
    PREFETCH = "prefetch"
    SHUTDOWN = "shutdown"


@dataclass
class KVRequest:
    request_type: KVRequestType
    request_id: int
    token_ids: np.ndarray
    token_mask: Optional[np.ndarray]
    slot_mapping: Optional[np.ndarray]
    layer_granularity: int = -1
    dp_id: int = 0


class KVResponseStatus(Enum):
    SUCCESS = "success"
    NOTFOUND = "not_found"
    UNREADY = "unready"
    TIMEOUT = "timeout"
    CANCELLED = "cancelled"
    FAILED = "failed"


@dataclass
class KVResponse:
    status: KVResponseStatus
    task_id: int
    return_mask: Optional[Union[np.ndarray, List[np.ndarray]]]

    def get_mask(self, idx: int) -> torch.Tensor:
        assert isinstance(self.return_mask, list), "return_mask is not a list of masks"
        return torch.from_numpy(self.return_mask[idx])
