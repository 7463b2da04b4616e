"""Records the TensorRT-LLM connector keeps per request and hands to the worker side
(flexkv/integration/tensorrt_llm/meta.py:9-89)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .utils import RequestWrapper


@dataclass
class FlexKVConnectorMetadata:
    """What ``build_connector_meta`` gives the workers each step: requests whose offload / restore ended."""
    finished_sending: List[str] = field(default_factory=list)
    finished_recving: List[str] = field(default_factory=list)

    def __getitem__(self, key: str):          # also readable as a mapping
        return set(getattr(self, key))


@dataclass
class FlexKVResponse:
    task_id: int
    task_type: str              # "get" | "put"
    request: RequestWrapper
    success: bool


@dataclass
class FlexKVTask:
    task_id: int
    request: RequestWrapper
    task_type: str = "get"
    slot_mapping: Optional[np.ndarray] = None
    num_computed_tokens: int = 0
    num_new_matched_tokens: int = 0
    num_unmatched_tokens: int = 0
    match_start_time: float = 0.0
    match_end_time: float = 0.0
    task_launch_time: float = 0.0
    task_finished_time: float = 0.0

    @property
    def match_cost(self) -> float:
        return self.match_end_time - self.match_start_time

    @property
    def task_execute_cost(self) -> float:
        return self.task_finished_time - self.task_launch_time

    def launched(self) -> None:
        self.task_launch_time = time.perf_counter()

    def finished(self) -> None:
        self.task_finished_time = time.perf_counter()

    def __str__(self) -> str:
        return (f"FlexKV{self.task_type.capitalize()}Task(task_id={self.task_id}, request={self.request.req_id}, "
                f"match {self.match_cost * 1e3:.2f} ms, execute {self.task_execute_cost * 1e3:.2f} ms)")
