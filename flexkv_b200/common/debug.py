"""Logging helpers: one package logger honouring ``FLEXKV_LOG_LEVEL`` and
``FLEXKV_LOGGING_PREFIX``, structured ``key=value`` operation logs, an eviction
log aggregator and a timing decorator (flexkv/common/debug.py:129-283,360;
csrc/logging.cpp:50-104)."""
from __future__ import annotations

import functools
import logging
import os
import threading
import time
from typing import Any, Callable, Dict, Optional

_LEVELS = {"TRACE": 5, "DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARN": logging.WARNING,
           "WARNING": logging.WARNING, "ERROR": logging.ERROR, "CRITICAL": logging.CRITICAL, "OFF": 100}


def _make_logger() -> logging.Logger:
    lg = logging.getLogger("flexkv")
    if not lg.handlers:
        h = logging.StreamHandler()
        prefix = os.getenv("FLEXKV_LOGGING_PREFIX", "FLEXKV")
        h.setFormatter(logging.Formatter(f"[{prefix}] %(levelname)s %(asctime)s.%(msecs)03d "
                                         f"[%(filename)s:%(lineno)d] %(message)s", "%m-%d %H:%M:%S"))
        lg.addHandler(h)
        lg.propagate = False
    lg.setLevel(_LEVELS.get(os.getenv("FLEXKV_LOG_LEVEL", "INFO").upper(), logging.INFO))
    return lg


flexkv_logger = _make_logger()


def set_log_level(level: str) -> None:
    flexkv_logger.setLevel(_LEVELS.get(level.upper(), logging.INFO))


def format_op_log(operation: str, act: str, status: str, **kv: Any) -> str:
    """``operation=put act=launch status=ok task_id=3 ...``"""
    parts = [f"operation={operation}", f"act={act}", f"status={status}"]
    parts += [f"{k}={v}" for k, v in kv.items()]
    return " ".join(parts)


def log_op(operation: str, act: str, status: str, level: int = logging.DEBUG, **kv: Any) -> None:
    if flexkv_logger.isEnabledFor(level):
        flexkv_logger.log(level, format_op_log(operation, act, status, **kv))


class EvictionLogAggregator:
    """Batches eviction events so a storm of small evictions prints one line per interval."""

    def __init__(self, interval_s: Optional[float] = None) -> None:
        if interval_s is None:          # FLEXKV_EVICTION_LOG_INTERVAL_S (flexkv/common/debug.py:150-160)
            try:
                interval_s = float(os.environ.get("FLEXKV_EVICTION_LOG_INTERVAL_S", "10"))
            except ValueError:
                interval_s = 10.0
            interval_s = max(0.1, interval_s)
        self.interval_s = float(interval_s)
        self._lock = threading.Lock()
        self._counts: Dict[str, int] = {}
        self._events: Dict[str, int] = {}
        self._last = time.monotonic()

    def record(self, tier: str, num_blocks: int) -> Optional[str]:
        with self._lock:
            self._counts[tier] = self._counts.get(tier, 0) + int(num_blocks)
            self._events[tier] = self._events.get(tier, 0) + 1
            now = time.monotonic()
            if now - self._last < self.interval_s:
                return None
            self._last = now
            msg = " ".join(f"{t}:blocks={self._counts[t]},events={self._events[t]}" for t in sorted(self._counts))
            self._counts.clear()
            self._events.clear()
        line = format_op_log("evict", "aggregate", "ok", detail=msg)
        flexkv_logger.info(line)
        return line

    def flush(self) -> Optional[str]:
        with self._lock:
            if not self._counts:
                return None
            msg = " ".join(f"{t}:blocks={self._counts[t]},events={self._events[t]}" for t in sorted(self._counts))
            self._counts.clear()
            self._events.clear()
        line = format_op_log("evict", "aggregate", "ok", detail=msg)
        flexkv_logger.info(line)
        return line


def debug_timing(name: Optional[str] = None) -> Callable:
    def deco(fn: Callable) -> Callable:
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def wrapper(*a: Any, **k: Any) -> Any:
            if not flexkv_logger.isEnabledFor(logging.DEBUG):
                return fn(*a, **k)
            t0 = time.perf_counter()
            try:
                return fn(*a, **k)
            finally:
                flexkv_logger.debug("%s took %.3f ms", label, (time.perf_counter() - t0) * 1e3)
        return wrapper
    return deco


_crash_diagnostics_installed = False


def install_crash_diagnostics(dump_signal: Optional[int] = None) -> bool:
    """On a fatal signal (SIGSEGV, SIGFPE, SIGABRT, SIGBUS, SIGILL) the interpreter prints the Python stack
    of every thread before it dies, and ``SIGUSR1`` (or ``dump_signal``) prints them on demand without
    stopping the process: the first thing wanted from a worker that crashed inside native code or sits
    in a call that never returns (flexkv/common/debug.py:315-337). Idempotent; returns False when the
    standard error stream has no file descriptor to write to."""
    global _crash_diagnostics_installed
    import faulthandler
    import signal
    import sys
    if _crash_diagnostics_installed:
        return True
    try:
        faulthandler.enable(file=sys.stderr, all_threads=True)
        sig = signal.SIGUSR1 if dump_signal is None else dump_signal
        faulthandler.register(sig, file=sys.stderr, all_threads=True, chain=False)
    except (ValueError, OSError, AttributeError, RuntimeError):
        return False
    _crash_diagnostics_installed = True
    return True
