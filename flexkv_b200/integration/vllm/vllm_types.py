"""Metadata and stats records of the vLLM connector as subclasses of vLLM's own base classes.

Imported only when vLLM is importable (``vllm_v1_adapter._vllm_types``): vLLM's scheduler output carries a
``KVConnectorMetadata``, its logger aggregates ``KVConnectorStats`` objects that travel between processes, so
both must be real, module-level (picklable) subclasses
(reference: flexkv/integration/vllm/vllm_v1_adapter.py:27-87,1159-1202).
"""
from dataclasses import dataclass

from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorMetadata

try:
    from vllm.distributed.kv_transfer.kv_connector.v1.metrics import KVConnectorStats
except Exception:  # noqa: BLE001 - vLLM older than its stats interface
    KVConnectorStats = None


class FlexKVConnectorMetadata(KVConnectorMetadata):
    """What the scheduler side did in this step. The workers have nothing to execute (the data plane moves the
    bytes), so the record only carries the request ids whose transfers finished."""

    def __init__(self, finished_sending=(), finished_recving=()) -> None:
        self.finished_sending = set(finished_sending)
        self.finished_recving = set(finished_recving)

    def __getitem__(self, key):
        return {"finished_sending": self.finished_sending, "finished_recving": self.finished_recving}[key]


if KVConnectorStats is not None:
    @dataclass
    class FlexKVConnectorStats(KVConnectorStats):
        """Counters of one interval: a dataclass holding one dict, like vLLM's own stats records."""

        def reset(self):
            self.data = {}

        def aggregate(self, other):
            for k, v in (getattr(other, "data", None) or {}).items():
                self.data[k] = self.data.get(k, 0) + v
            return self

        def reduce(self):
            d = dict(self.data)
            q = d.get("num_get_query_tokens", 0)
            if q:
                d["get_gpu_match_ratio"] = d.get("num_gpu_matched_tokens", 0) / q
                d["get_flexkv_match_ratio"] = d.get("num_flexkv_matched_tokens", 0) / q
            return d

        def is_empty(self) -> bool:
            """Nothing was counted in this interval: the engine's logger skips the record."""
            return not any(v for k, v in self.data.items() if not k.endswith("_ratio"))

        def __getitem__(self, key):
            return self.data[key]

    class FlexKVWorkerSentinelStats(KVConnectorStats):
        """What the worker side returns: it counts nothing itself, but a stats object that is not None keeps the
        worker's connector output from being dropped as empty, so the engine keeps asking the scheduler side for
        finished transfers on steps that schedule no tokens. Aggregation hands back the other side's record
        (reference: flexkv/integration/vllm/vllm_v1_adapter.py:66-82)."""

        def aggregate(self, other):
            return other

        def reduce(self):
            return {}

        def reset(self):
            pass

        def is_empty(self) -> bool:
            return True
else:
    FlexKVConnectorStats = None
    FlexKVWorkerSentinelStats = None
