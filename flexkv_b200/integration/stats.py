"""Per-adapter hit statistics (flexkv/integration/stats.py:11-99)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..common.debug import flexkv_logger


@dataclass
class FlexKVStats:
    log_interval: int = 100
    num_get_requests: int = 0
    num_get_query_tokens: int = 0
    num_gpu_matched_tokens: int = 0
    num_flexkv_matched_tokens: int = 0
    num_put_requests: int = 0
    num_put_query_tokens: int = 0
    num_put_unmatched_tokens: int = 0
    num_failed_requests: int = 0
    _t0: float = field(default_factory=time.monotonic)

    def record_get(self, num_total_tokens: int, num_gpu_matched: int, num_flexkv_matched: int) -> None:
        self.num_get_requests += 1
        self.num_get_query_tokens += num_total_tokens
        self.num_gpu_matched_tokens += num_gpu_matched
        self.num_flexkv_matched_tokens += num_flexkv_matched
        if self.log_interval and self.num_get_requests % self.log_interval == 0:
            self.log()

    def record_put(self, num_total_tokens: int, num_unmatched: int) -> None:
        self.num_put_requests += 1
        self.num_put_query_tokens += num_total_tokens
        self.num_put_unmatched_tokens += num_unmatched

    def record_failed(self, n: int = 1) -> None:
        self.num_failed_requests += n

    @property
    def flexkv_hit_ratio(self) -> float:
        return self.num_flexkv_matched_tokens / max(1, self.num_get_query_tokens)

    @property
    def gpu_hit_ratio(self) -> float:
        return self.num_gpu_matched_tokens / max(1, self.num_get_query_tokens)

    def log(self) -> None:
        flexkv_logger.info("[stats] gets=%d query_tok=%d gpu_hit=%.1f%% flexkv_hit=%.1f%% puts=%d put_new_tok=%d "
                           "failed=%d", self.num_get_requests, self.num_get_query_tokens, 100 * self.gpu_hit_ratio,
                           100 * self.flexkv_hit_ratio, self.num_put_requests, self.num_put_unmatched_tokens,
                           self.num_failed_requests)
