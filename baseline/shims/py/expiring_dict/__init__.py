"""Stand-in for the ``expiring-dict`` package (absent from this image): a thread-safe dict whose
entries may carry a time-to-live. Constructor keywords the reference passes are accepted."""
import threading
import time


class ExpiringDict(dict):
    def __init__(self, ttl=None, interval=0.1, max_age_seconds=None, max_len=None):
        super().__init__()
        self._ttl = ttl if ttl is not None else max_age_seconds
        self._max_len = max_len
        self._born = {}
        self._lock = threading.RLock()

    def __class_getitem__(cls, item):
        return cls

    def _purge(self):
        if self._ttl is None or not self._born:
            return
        now = time.monotonic()
        dead = [k for k, t in list(self._born.items()) if now - t > self._ttl]
        for k in dead:
            self._born.pop(k, None)
            super().pop(k, None)

    def __setitem__(self, key, value):
        with self._lock:
            if self._ttl is not None:
                if len(self._born) >= 4096 and len(self._born) % 1024 == 0:
                    self._purge()
                self._born[key] = time.monotonic()
            super().__setitem__(key, value)

    def __delitem__(self, key):
        with self._lock:
            self._born.pop(key, None)
            super().__delitem__(key)

    def pop(self, key, *default):
        with self._lock:
            self._born.pop(key, None)
            return super().pop(key, *default)

    def ttl(self, key, value, ttl):
        self[key] = value
