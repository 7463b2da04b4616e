"""The registry's command set over the Redis wire protocol.

``RedisRegistryClient`` has the methods of ``registry.RegistryClient`` (incr, hset, hset_many, hgetall,
expire, exists, delete, scan, scan_values, delete_prefix), so ``NodeRegistry`` and ``RegistryMetaChannel``
run unchanged against a Redis server: the same key schema as the reference keeps there
(flexkv/cache/redis_meta.py:158-906, csrc/dist/redis_meta_channel.cpp:198-215). The protocol is spoken by
the native ``RespClient``; commands that touch many keys are pipelined.
"""
from __future__ import annotations

import re
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

_INT = re.compile(rb"^-?\d{1,20}$")
_FLOAT = re.compile(rb"^-?\d+\.\d*(e[+-]?\d+)?$|^-?\d+e[+-]?\d+$", re.I)


def _decode(v: bytes) -> Any:
    """Redis stores strings; numbers written through ``hset`` come back as numbers."""
    if _INT.match(v):
        return int(v)
    if _FLOAT.match(v):
        return float(v)
    return v.decode("utf-8", "surrogateescape")


def _encode(v: Any) -> bytes:
    if isinstance(v, bytes):
        return v
    if isinstance(v, bool):
        return b"1" if v else b"0"
    if isinstance(v, float):
        return repr(v).encode()
    return str(v).encode("utf-8", "surrogateescape")


def _glob_escape(prefix: str) -> str:
    return re.sub(r"([*?\[\]\\])", r"\\\1", prefix)


class RedisRegistryClient:
    def __init__(self, host: str, port: int = 6379, password: str = "", db: int = 0, timeout_ms: int = 3000) -> None:
        from .. import _native
        self._addr = (host, int(port), int(timeout_ms), password or "", int(db))
        self._c = _native.C.RespClient(host, int(port), int(timeout_ms), password or "", int(db))

    def native_channel(self, kind: str = "CPUB"):
        """The block-record channel of the cross-node index over its own connection, served from native code
        (the trees' refresh threads then never take the interpreter lock for it)."""
        from .. import _native
        host, port, timeout_ms, password, db = self._addr
        return _native.C.RedisMetaChannel(host, port, kind, timeout_ms, password, db)

    def close(self) -> None:
        self._c.close()

    def ping(self) -> bool:
        return self._c.command("PING") == "PONG"

    # ---- the registry's commands -------------------------------------------------------
    def incr(self, key: str) -> int:
        return int(self._c.command("INCR", key))

    @staticmethod
    def _hset_cmd(key: str, mapping: Dict[str, Any]) -> List[Any]:
        cmd: List[Any] = ["HSET", key]
        for f, v in mapping.items():
            cmd += [str(f), _encode(v)]
        return cmd

    def hset(self, key: str, mapping: Dict[str, Any], ttl: Optional[float] = None, only_if_exists: bool = False) -> bool:
        if only_if_exists and not self.exists(key):
            return False
        cmds = [self._hset_cmd(key, mapping)]
        if ttl is not None:
            cmds.append(["PEXPIRE", key, max(1, int(ttl * 1000))])
        self._c.pipeline(cmds)
        return True

    def hset_many(self, items: Sequence[Tuple[str, Dict[str, Any]]]) -> int:
        if items:
            self._c.pipeline([self._hset_cmd(k, m) for k, m in items])
        return len(items)

    @staticmethod
    def _pairs(flat) -> Dict[str, Any]:
        return {flat[i].decode(): _decode(flat[i + 1]) for i in range(0, len(flat or ()), 2)}

    def hgetall(self, key: str) -> Dict[str, Any]:
        return self._pairs(self._c.command("HGETALL", key))

    def expire(self, key: str, ttl: float) -> bool:
        """PEXPIRE answers 0 for a key that is gone: an expired node is never resurrected."""
        return int(self._c.command("PEXPIRE", key, max(1, int(ttl * 1000)))) == 1

    def exists(self, key: str) -> bool:
        return int(self._c.command("EXISTS", key)) > 0

    def delete(self, keys: Iterable[str]) -> int:
        keys = list(keys)
        n = 0
        for i in range(0, len(keys), 512):
            n += int(self._c.command("DEL", *keys[i:i + 512]))
        return n

    def scan(self, prefix: str) -> List[str]:
        out, cursor = set(), "0"
        pattern = _glob_escape(prefix) + "*"
        while True:
            cursor, keys = self._c.command("SCAN", cursor, "MATCH", pattern, "COUNT", 1000)
            out.update(k.decode() for k in keys)
            cursor = cursor.decode() if isinstance(cursor, bytes) else str(cursor)
            if cursor == "0":
                return sorted(out)

    def scan_values(self, prefix: str) -> List[Dict[str, Any]]:
        keys = self.scan(prefix)
        if not keys:
            return []
        rows = self._c.pipeline([["HGETALL", k] for k in keys])
        return [d for d in (self._pairs(r) for r in rows) if d]          # a key may have expired since the scan

    def delete_prefix(self, prefix: str) -> int:
        return self.delete(self.scan(prefix))
