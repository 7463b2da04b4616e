"""Per-op transfer trace: ``[XFER]`` lines with queue wait, transfer time and
bandwidth, and a periodic ``[XFER-SUMMARY]`` with p50/p99 per op type
(enabled by ``FLEXKV_TRANSFER_TRACE=1``; reference: flexkv/transfer/trace.py:134-199)."""
from __future__ import annotations

import threading
import time
from collections import defaultdict
from typing import Dict, List

from ..common.debug import flexkv_logger


def _pct(v: List[float], q: float) -> float:
    if not v:
        return 0.0
    s = sorted(v)
    return s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))]


class TransferTrace:
    def __init__(self, enabled: bool = False, summary_interval_s: float = 10.0) -> None:
        self.enabled = enabled
        self.summary_interval_s = summary_interval_s
        self._t_submit: Dict[int, float] = {}
        self._samples: Dict[str, List[float]] = defaultdict(list)
        self._bw: Dict[str, List[float]] = defaultdict(list)
        self._last_summary = time.monotonic()
        self._lock = threading.Lock()
        self.lines: List[str] = []      # kept for tests and post-mortems (bounded)

    def on_submit(self, op) -> None:
        if self.enabled:
            self._t_submit[op.op_id] = time.perf_counter()

    def on_done(self, op, outcome) -> None:
        if not self.enabled:
            return
        t0 = self._t_submit.pop(op.op_id, None)
        e2e_ms = (time.perf_counter() - t0) * 1e3 if t0 is not None else 0.0
        xfer_ms = outcome.gpu_ms if outcome.gpu_ms > 0 else e2e_ms
        bw = outcome.num_bytes / (xfer_ms * 1e-3) / 1e9 if xfer_ms > 0 else 0.0
        line = (f"[XFER] op={op.op_id} type={op.transfer_type.value} blocks={op.valid_block_num} "
                f"bytes={outcome.num_bytes} wait_ms={max(0.0, e2e_ms - xfer_ms):.3f} xfer_ms={xfer_ms:.3f} "
                f"e2e_ms={e2e_ms:.3f} bw_GBps={bw:.2f} ok={int(outcome.success)}")
        with self._lock:
            self.lines.append(line)
            del self.lines[:-1000]
            self._samples[op.transfer_type.value].append(e2e_ms)
            self._bw[op.transfer_type.value].append(bw)
        flexkv_logger.info(line)
        if time.monotonic() - self._last_summary >= self.summary_interval_s:
            self.summary()

    def summary(self) -> List[str]:
        out = []
        with self._lock:
            self._last_summary = time.monotonic()
            for tt, v in self._samples.items():
                out.append(f"[XFER-SUMMARY] type={tt} n={len(v)} p50_ms={_pct(v, 0.5):.3f} p99_ms={_pct(v, 0.99):.3f} "
                           f"bw_p50_GBps={_pct(self._bw[tt], 0.5):.2f}")
            self._samples.clear()
            self._bw.clear()
        for l in out:
            flexkv_logger.info(l)
        return out
